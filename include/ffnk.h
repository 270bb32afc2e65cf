/*
 * ffnk.h -- C ABI of the B200 (sm_100a) routed MaskedLinear / MaskedFFN kernels.
 *
 * Plain pointers and sizes only.  Every pointer is a DEVICE pointer on the current CUDA
 * device unless stated otherwise; `stream` is a cudaStream_t passed as void*.  Nothing here
 * allocates or synchronises unless its comment says so: the caller owns every buffer
 * (outputs, routing lists, scratch) and orders work by stream.
 *
 * Return value: 0 on success; a negative FFNK_ERR_* for a rejected argument (nothing was
 * launched); -(1000 + cudaError_t) for a CUDA runtime error reported at launch.  Device-side
 * protocol errors (a bounded wait that expired) are written as small positive codes to the
 * int32 status word the caller passes and read back with ffnk_read_status().
 *
 * Citations are file:line in the reference project (wenhaoli-xmu/ffn_kernel) whose host
 * launchers these entry points replace.
 *
 * Conventions shared by all entry points
 *   - Activations are bf16, row-major with an element row stride (`ld*`), 16-byte aligned rows.
 *   - A weight is the logical [K, N] matrix the reference's operators receive (b1/b2, w*, u*).
 *     It is described by its element strides (stride_k, stride_n); exactly one of them must
 *     be 1.  stride_k == 1 is the `nn.Linear.weight.T` view (storage [N, K]); stride_n == 1
 *     is a contiguous [K, N] matrix.  This library never copies or transposes a weight; all
 *     weights of one call share one pair of strides (anything else is the caller's to repack).
 *   - mask: one byte per token, non-zero = first weight set ("visual"), zero = second ("text")
 *     (ffn_kernel/linear.py:137-140).
 *   - Routing lists (`perm`, `counts`) are produced by ffnk_route() on the same stream.
 *   - The GEMM entry points encode TMA tensor maps on the host through the driver, which needs the
 *     device's primary context bound to the calling thread; the first such call on a thread binds it
 *     (cudaFree(0)).  Make a thread's first call outside any stream capture; later calls can be captured.
 */
#ifndef FFNK_H_
#define FFNK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FFNK_ERR_NULL (-1)      /* a required pointer is null */
#define FFNK_ERR_SHAPE (-2)     /* a size is negative, too large or not a multiple of 8 */
#define FFNK_ERR_ALIGN (-3)     /* a base pointer or row stride is not 16-byte aligned */
#define FFNK_ERR_LAYOUT (-4)    /* a weight has neither stride_k == 1 nor stride_n == 1 */
#define FFNK_ERR_DRIVER (-5)    /* the CUDA driver entry point for tensor maps is unavailable */
#define FFNK_ERR_TENSORMAP (-6) /* the driver rejected a tensor map */
#define FFNK_ERR_DEVICE (-7)    /* the current device is not compute capability 10.x */
#define FFNK_ERR_CAPACITY (-8)  /* the problem exceeds the fixed capacity of a no-allocation entry point */
#define FFNK_ERR_CAPTURE (-9)   /* first call of a no-allocation entry point on this device made during stream capture */

/* Library version (major * 100 + minor). */
int ffnk_version(void);

/* ---------------------------------------------------------------------------------------
 * Routing.  No counterpart as a function in the reference: it replaces the per-tile
 * uniformity test of every reference kernel (ffn_kernel/linear.py:132,137;
 * ffn_kernel/ffn.py:72,79) by explicit per-modality row lists.
 *
 *   cap  = ffnk_route_capacity(M)           (M rounded up to a multiple of 128)
 *   perm   int32[2 * cap], 16-byte aligned: perm[0..Mv) ascending visual rows,
 *                                           perm[cap..cap+Mt) ascending text rows
 *   counts int32[8] = { Mv, Mt, cap, M, runs, -, -, - }   (stay on the device; no host sync)
 *          runs = number of maximal stretches of consecutive same-modality tokens
 *   workspace: ffnk_route_workspace_bytes(M) bytes, cleared by the call itself
 * Masks of more than 2^20 tokens whose bits fit in the GPU's shared memory (one bit per token; 2^26
 * tokens are 8 MiB) are routed by ONE kernel whose CTAs wait for one another once: the barrier-counter
 * rule of ffnk_ffn_decode applies to it (its counters are this library's own, one per launch in turn
 * over 64 slots; a grid that is not resident all at once reports the status "grid-wide wait expired"
 * instead of hanging), and its first call on a process queries the occupancy of that kernel: make it
 * outside any stream capture.
 * ------------------------------------------------------------------------------------- */
int64_t ffnk_route_capacity(int64_t M);
int64_t ffnk_route_workspace_bytes(int64_t M);
int ffnk_route(const void* mask, int64_t M, int32_t* perm, int32_t* counts, void* workspace, int32_t* status,
               void* stream);

/* ---------------------------------------------------------------------------------------
 * Routing for callers that cannot provide scratch memory.  This entry point has no counterpart
 * in the reference; it exists for hosts that must not allocate when they call: a serving-runtime
 * plugin whose execute callback gets every buffer up front and may not allocate device memory,
 * or a steady-state loop that avoids cudaMalloc because it synchronises the device.
 *
 * Same results as ffnk_route() (perm, counts as described above) but without the workspace
 * argument: the scan state lives in a fixed 8.25 KiB array inside the library, which every GPU
 * that loads the library keeps until the process exits.  Consequences:
 *   - M may not exceed FFNK_ROUTE_NOALLOC_MAX_TOKENS; a longer mask returns FFNK_ERR_CAPACITY
 *     and launches nothing.
 *   - All calls on a device share that one array (each call clears the part it uses), so two
 *     calls that may run on the GPU at the same time -- different streams -- race.  Issue them
 *     on one stream, or order them with events.
 *   - The first call on each device looks up the array's device address; make that first call
 *     outside any stream capture (an empty mask will not do: it returns before the lookup).  A first
 *     call that arrives while `stream` is being captured returns FFNK_ERR_CAPTURE and launches nothing.
 *     Nothing is allocated or freed, then or later.
 * ------------------------------------------------------------------------------------- */
#define FFNK_ROUTE_NOALLOC_MAX_TOKENS 16777216 /* 2^24 tokens */
int ffnk_route_noalloc(const void* mask, int64_t M, int32_t* perm, int32_t* counts, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * MaskedLinear forward.  Replaces _bf16_linear_forward (ffn_kernel/linear.py:418-452) and
 * the kernel it launches (_masked_matmul_infer, ffn_kernel/linear.py:76-159):
 *     c[m, :] = a[m, :] @ (mask[m] ? b1 : b2)        a [M,K], b* [K,N], c [M,N] bf16
 * bf16 operands, fp32 accumulation, bf16 output.  Every row of c is written exactly once.
 * a_copy: optional scratch bf16 [(cap + 512), K], or null.  Token rows are normally gathered by
 * the GEMM itself (tiled TMA boxes for runs of consecutive tokens, gather4 for ragged rows); with
 * the scratch, a mask whose runs average under max(32, N / 6) tokens (decided on the device from
 * counts[4]) makes the call copy a into routed order first and read that instead: 2.7x faster on
 * i.i.d. masks, a few percent on 576-token spans at N = 4096.
 * ------------------------------------------------------------------------------------- */
int ffnk_linear_fwd(const void* a, int64_t lda, const void* b1, const void* b2, int64_t b_stride_k,
                    int64_t b_stride_n, const int32_t* perm, const int32_t* counts, void* c, int64_t ldc, void* a_copy,
                    int64_t M, int64_t N, int64_t K, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * MaskedLinear backward.  Replaces _bf16_linear_backward (ffn_kernel/linear.py:455-496) and
 * _fused_bwd_kernel / _masked_matmul_bwd_da / _masked_matmul_bwd_db
 * (ffn_kernel/linear.py:15-72, 242-326, 329-415):
 *     da[m, :] = g[m, :] @ (mask[m] ? b1 : b2)^T
 *     db1 = a[mask]^T @ g[mask],   db2 = a[~mask]^T @ g[~mask]
 * db1/db2 are written with the same strides as b1/b2 (the reference allocates them with
 * empty_like, ffn_kernel/linear.py:475).
 * g_copy [(cap + 512), N], a_copy [(cap + 512), K]: optional scratch (both or neither).  With it
 * the call first copies g and a into routed order (for every mask) and all three GEMMs read whole
 * tiles of consecutive rows: dx with the kernel of ffnk_ffn_down, the weight gradients on CTA
 * pairs (M=32768, K=N=4096: 1.82 ms against 2.12-2.29 ms without).  Without it the kernels
 * gather token rows themselves; worthwhile only for small M.
 * a may be null when both scratch matrices are given and a_copy already holds a in routed order
 * (ffnk_permute_rows in the forward pass, which can then run its GEMM as ffnk_ffn_down on that copy):
 * the call then skips that copy.
 * ------------------------------------------------------------------------------------- */
int ffnk_linear_bwd(const void* g, int64_t ldg, const void* a, int64_t lda, const void* b1, const void* b2,
                    int64_t b_stride_k, int64_t b_stride_n, const int32_t* perm, const int32_t* counts, void* da,
                    int64_t ldda, void* db1, void* db2, void* g_copy, void* a_copy, int64_t M, int64_t N, int64_t K,
                    int32_t* status, void* stream);

/* The same in separately callable parts, for data-parallel training (no counterpart in the single-device
 * reference): parts is a bit mask, 1 = the routed-order copies of g and a, 2 = the weight gradients,
 * 4 = dx.  ffnk_linear_bwd is parts = 7.  A caller that sums weight gradients over ranks runs 1|2,
 * starts the all-reduce of db1/db2 on another stream, and runs 4 on this stream beside it. */
int ffnk_linear_bwd_parts(const void* g, int64_t ldg, const void* a, int64_t lda, const void* b1, const void* b2,
                          int64_t b_stride_k, int64_t b_stride_n, const int32_t* perm, const int32_t* counts, void* da,
                          int64_t ldda, void* db1, void* db2, void* g_copy, void* a_copy, int64_t M, int64_t N,
                          int64_t K, int parts, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Copies the rows of x [M, d] into routed order: out [(cap + 512), d], visual rows first, text
 * rows from row 256 * ceil(Mv / 256).  No counterpart in the reference (it never reorders
 * tokens); used in front of ffnk_ffn_gateup(routed_in = 1) when one extra pass over x is
 * cheaper than gathering ragged rows inside the GEMM.
 * ------------------------------------------------------------------------------------- */
int ffnk_permute_rows(const void* x, int64_t ldx, const int32_t* perm, const int32_t* counts, void* out, int64_t ldo,
                      int64_t M, int64_t d, void* stream);

/* ffnk_route followed by ffnk_permute_rows in ONE launch, for masks of at most
 * ffnk_route_permute_max_tokens() (8192) tokens: every CTA routes the whole mask for itself in shared memory
 * and copies its share of the rows; perm and counts come out as from ffnk_route.  Needs no workspace and
 * reports no device status (nothing in it waits).  The MaskedFFN forward uses it below that size whenever
 * it copies x first. */
int64_t ffnk_route_permute_max_tokens(void);
int ffnk_route_permute_rows(const void* mask, int64_t M, const void* x, int64_t ldx, int64_t d, int32_t* perm,
                            int32_t* counts, void* out, int64_t ldo, void* stream);

/* ---------------------------------------------------------------------------------------
 * MaskedFFN gate/up projection with the SwiGLU epilogue.  Replaces _bf16_ffn_forward
 * (ffn_kernel/ffn.py:527-560) and _masked_ffn_infer (ffn_kernel/ffn.py:15-113):
 *     t1 = x @ (mask ? w1 : u1),  t3 = x @ (mask ? w3 : u3),  out = silu(t1) * t3
 * x [M,d]; w1,w3,u1,u3 [d,h] sharing one pair of strides; out bf16.
 *   routed_in  == 0: x is [M, d] in token order; its rows are gathered by the kernel.
 *   routed_in  != 0: x is [(cap + 512), d] already in routed order (ffnk_permute_rows).
 *   routed_out == 0: out is [M, h] in token order (what the reference function returns).
 *   routed_out != 0: out is the routed intermediate [(cap + 512), h]: visual rows first,
 *                    text rows from row 256 * ceil(Mv / 256); rows in between are not written.
 * ------------------------------------------------------------------------------------- */
int ffnk_ffn_gateup(const void* x, int64_t ldx, const void* w1, const void* w3, const void* u1, const void* u3,
                    int64_t w_stride_k, int64_t w_stride_n, const int32_t* perm, const int32_t* counts, void* out,
                    int64_t ldo, int routed_in, int routed_out, int64_t M, int64_t d, int64_t h, int32_t* status,
                    void* stream);

/* ---------------------------------------------------------------------------------------
 * MaskedFFN down projection from the routed intermediate, rows scattered back to token order
 * in the epilogue.  Together with ffnk_ffn_gateup(routed_out = 1) this replaces
 * MaskedFFN.forward (ffn_kernel/ops.py:28-32), whose second step is _bf16_linear_forward on
 * the intermediate:
 *     y[token, :] = inter[routed row of token, :] @ (mask[token] ? w2 : u2)
 * inter [(cap + 512), h] as written by ffnk_ffn_gateup; w2,u2 [h,d]; y [M,d] bf16.
 * ------------------------------------------------------------------------------------- */
int ffnk_ffn_down(const void* inter, int64_t ldi, const void* w2, const void* u2, int64_t w_stride_k,
                  int64_t w_stride_n, const int32_t* perm, const int32_t* counts, void* y, int64_t ldy, int64_t M,
                  int64_t d, int64_t h, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Tensor parallel over h: down projection fused with the first half of a reduce-scatter.
 * The reference is single-device (test_linear.py:74 selects device 0); this has no counterpart
 * there.  Each of `world` ranks holds h / world columns of the intermediate and the matching rows
 * of w2/u2, so its down projection is a partial sum of every output row.  Token t is owned by
 * rank t / rows_per_rank.  Instead of writing its partial y and handing it to a collective, the
 * GEMM's epilogue stores each partial row directly into the owner's memory over NVLink:
 *     peer_blocks[t / rows_per_rank][(rank * rows_per_rank + t % rows_per_rank) * ldb + c]
 *         = partial y[t, c]
 * peer_blocks is a HOST array of `world` device pointers (1 <= world <= 8): entry r is rank r's
 * block buffer, bf16 [world * rows_per_rank, ldb], mapped into this process (CUDA IPC, a
 * symmetric-memory allocation, or cudaMalloc'd memory of a peer-enabled device in the same
 * process); entry `rank` is this rank's own buffer.  rows_per_rank * world >= M.
 * The call does not wait for or signal other ranks: the caller orders it after every owner has
 * finished reading the previous contents of its buffer, and orders ffnk_sum_row_blocks on each
 * owner after all ranks' calls have completed (a stream-ordered barrier between the two).
 * ------------------------------------------------------------------------------------- */
int ffnk_ffn_down_to_peers(const void* inter, int64_t ldi, const void* w2, const void* u2, int64_t w_stride_k,
                           int64_t w_stride_n, const int32_t* perm, const int32_t* counts,
                           void* const* peer_blocks, int world, int rank, int64_t rows_per_rank, int64_t ldb,
                           int64_t M, int64_t d, int64_t h, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * Second half of that reduce-scatter, run by the owner on its own buffer:
 *     out[r, c] = bf16( sum over b < nblocks of fp32(blocks[(b * rows + r) * ldb + c]) )
 * blocks bf16 [nblocks * rows, ldb]; out bf16 [rows, ldo]; d columns, d % 8 == 0.
 * No counterpart in the reference.
 * ------------------------------------------------------------------------------------- */
int ffnk_sum_row_blocks(const void* blocks, int nblocks, int64_t rows, int64_t d, int64_t ldb, void* out,
                        int64_t ldo, void* stream);

/* ---------------------------------------------------------------------------------------
 * The rest of the tensor-parallel all-reduce with this library's own kernels (no counterpart in the
 * single-device reference).  After ffnk_ffn_down_to_peers on every rank:
 *     ffnk_peer_barrier            every rank's partial rows have landed in their owners' buffers
 *     ffnk_sum_row_blocks_to_peers the owner sums its `nblocks` blocks (block_rows rows apart; the first
 *                                  `rows` <= block_rows rows of each) in fp32 and stores the bf16 rows into
 *                                  the output matrix of EVERY rank: peer_out[r][(out_row0 + row) * ldo + c]
 *     ffnk_peer_barrier            every rank's output matrix is complete
 * flags / peer_out are HOST arrays of `world` device pointers (1 <= world <= 8), entry r belonging to
 * rank r and mapped into this process like peer_blocks above.  A flag array is int32[8], zeroed once
 * before its first use.  `epoch` is 1, 2, 3, ... and must be the same on all ranks for the same barrier
 * (every rank calls the barriers of one flag array in the same order).  The barrier kernel is one warp:
 * it release-stores `epoch` into slot `rank` of every rank's array, then polls its own array until every
 * slot has reached `epoch`; after budget_us microseconds (0: the library's 2 s) it gives up, writes a
 * status code to `status` and returns, so a missing rank surfaces in ffnk_read_status, not as a hang.
 * Ranks must be separate GPUs (kernels of different ranks waiting for each other on one GPU may never
 * run at the same time).  max_ctas > 0 caps the grid of the sum (to leave SMs to a concurrent GEMM).
 * ------------------------------------------------------------------------------------- */
int ffnk_peer_barrier(void* const* flags, int world, int rank, int32_t epoch, int64_t budget_us, int32_t* status,
                      void* stream);
int ffnk_sum_row_blocks_to_peers(const void* blocks, int nblocks, int64_t block_rows, int64_t rows, int64_t d,
                                 int64_t ldb, void* const* peer_out, int world, int64_t out_row0, int64_t ldo,
                                 int max_ctas, void* stream);

/* ---------------------------------------------------------------------------------------
 * Small-M (decode) MaskedFFN forward in one launch, bound by HBM bandwidth: one persistent kernel
 * streams each present modality's weights once with 128-bit loads (the down-projection rows prefetched
 * into L2 while gate/up runs), with a bounded grid-wide wait between the two phases.  Same contract as
 * MaskedFFN.forward (ffn_kernel/ops.py:28-32).  inter: scratch bf16 [M, h].  K-major weights only.
 * The grid-wide wait counts arrivals in one of 64 counters inside the library; successive launches take
 * successive counters and a launch captured into a CUDA graph keeps the one it was captured with, so two
 * launches that may run on the GPU at the same time must not be a multiple of 64 launches apart (launches
 * on one stream never overlap; graphs that replay concurrently should be captured back to back).
 * Accepts M <= ffnk_decode_capacity() (127).  ffnk_ffn_takes_decode(M, d, h) is the tile table's entry:
 * whether ffnk_ffn_forward sends this shape here (never beyond ffnk_decode_max_tokens() = 80 tokens;
 * wide FFNs switch to the GEMM path earlier, d=4096/h=11008 at 22 tokens, because every CTA re-reads
 * the token rows for each of its row blocks).
 * ------------------------------------------------------------------------------------- */
int ffnk_decode_max_tokens(void);
int ffnk_decode_capacity(void);
int ffnk_ffn_takes_decode(int64_t M, int64_t d, int64_t h);
int ffnk_ffn_decode(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3, const void* u1,
                    const void* u2, const void* u3, int64_t w13_stride_k, int64_t w13_stride_n, int64_t w2_stride_k,
                    int64_t w2_stride_n, const void* mask, void* inter, void* y, int64_t ldy, int64_t M, int64_t d,
                    int64_t h, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * The whole MaskedFFN forward in one call (MaskedFFN.forward, ffn_kernel/ops.py:28-32):
 * routing, optional row permutation, gate/up, down -- or the decode kernel when
 * allow_decode != 0, ffnk_ffn_takes_decode(M, d, h) and the weights are K-major.
 * workspace: ffnk_ffn_workspace_bytes(M, d, h) bytes of device memory, 256-byte aligned, owned by
 * the caller and reusable as soon as the stream has passed this call; too small a workspace
 * returns FFNK_ERR_CAPACITY.  ffnk_ffn_permute_first() tells whether the tile table copies x
 * into routed order first for this shape.
 * With few row tiles (up to 384 tokens at d = 1024, h = 2816) the down projection cuts its contraction
 * into ranges on different SMs; their arrival counters are this library's own, one row of counters per
 * launch in turn over 64 rows, each left at zero by the launch that used it: the barrier-counter rule
 * of ffnk_ffn_decode applies (no more than 64 such launches in flight on one device at a time; a
 * captured launch keeps the row it was captured with).  The result does not depend on which range
 * finishes last (the partial tiles are added in a fixed order).
 * ------------------------------------------------------------------------------------- */
int64_t ffnk_ffn_workspace_bytes(int64_t M, int64_t d, int64_t h);
int ffnk_ffn_permute_first(int64_t M, int64_t d, int64_t h);
int ffnk_ffn_forward(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3, const void* u1,
                     const void* u2, const void* u3, int64_t w13_stride_k, int64_t w13_stride_n, int64_t w2_stride_k,
                     int64_t w2_stride_n, const void* mask, void* workspace, int64_t workspace_bytes, void* y,
                     int64_t ldy, int64_t M, int64_t d, int64_t h, int allow_decode, int32_t* status, void* stream);

/* ---------------------------------------------------------------------------------------
 * MaskedFFN forward that keeps what the backward pass needs, and the backward pass.  The
 * reference has no working counterpart: its saving forward kernel (_masked_ffn_fwd,
 * ffn_kernel/ffn.py:116-221) is never launched, its backward kernels (ffn_kernel/ffn.py:224-524)
 * do not compile and MaskedFFN.backward raises (ffn_kernel/ops.py:34-38); the formulas are those
 * of the reference's README.md:159-172.
 *
 * rows = ffnk_route_capacity(M) + 512.  The caller owns, and keeps alive between the two calls:
 *   perm int32[2*cap], counts int32[8]      routing lists (written by the forward, as by ffnk_route)
 *   xr  bf16 [rows, d]                      x in routed order
 *   t1, t3, hid bf16 [rows, h]              gate and up pre-activations, and silu(t1) * t3
 * Backward scratch: gr bf16 [rows, d], dt1 and dt3 bf16 [rows, h].  The six weight gradients are
 * written with the strides of their weights; dx is [M, d] in token order.
 * ------------------------------------------------------------------------------------- */
int ffnk_ffn_forward_train(const void* x, int64_t ldx, const void* w1, const void* w2, const void* w3, const void* u1,
                           const void* u2, const void* u3, int64_t w13_stride_k, int64_t w13_stride_n,
                           int64_t w2_stride_k, int64_t w2_stride_n, const void* mask, int32_t* perm, int32_t* counts,
                           void* scan_workspace, void* xr, void* t1, void* t3, void* hid, void* y, int64_t ldy,
                           int64_t M, int64_t d, int64_t h, int32_t* status, void* stream);
int ffnk_ffn_backward(const void* gy, int64_t ldg, const void* xr, const void* t1, const void* t3, const void* hid,
                      const void* w1, const void* w2, const void* w3, const void* u1, const void* u2, const void* u3,
                      int64_t w13_stride_k, int64_t w13_stride_n, int64_t w2_stride_k, int64_t w2_stride_n,
                      const int32_t* perm, const int32_t* counts, void* gr, void* dt1, void* dt3, void* dx,
                      int64_t lddx, void* dw1, void* dw2, void* dw3, void* du1, void* du2, void* du3, int64_t M,
                      int64_t d, int64_t h, int32_t* status, void* stream);

/* Synchronises `stream`, copies the status word to the host and returns it (0 = ok, >0 one of
 * the device status codes, <0 an error as above).  If `clear` is non-zero the word is reset to 0. */
int ffnk_read_status(int32_t* status, int clear, void* stream);

/* Exercises the bounded-wait path on purpose: one CTA waits on a barrier nobody arrives on,
 * with a budget of `budget_us` microseconds, then records its status and exits normally.
 * Used by the tests to show that an expired wait surfaces as a status code. */
int ffnk_selftest_bounded_wait(int32_t* status, int64_t budget_us, void* stream);

/* The GEMM kernels are persistent and by default occupy every SM.  A caller that overlaps them
 * with a collective on another stream (tensor-parallel chunks) sets a margin so that many SMs stay
 * free for the collective's kernels; 0 restores the default.  Process-wide, affects later launches. */
int ffnk_set_sm_margin(int sms);

/* Diagnostics: when `buffer` (device memory, 8 int64 per CTA of the largest grid, i.e. 8 * SM count)
 * is non-null, the CTA-pair GEMM kernels launched afterwards store per-CTA cycle counters in it:
 * [0] MMA-issuer total, [1] its wait for operands, [2] its wait for a free accumulator,
 * [3] producer wait for a free stage, [4] producer total, [5] epilogue wait for an accumulator,
 * [6] epilogue total, [7] tiles.  The decode kernel stores cycle stamps since its start instead: [0] tokens
 * counted, [1] first gate/up weights requested, [2] gate/up done, [3] first down weights requested,
 * [4] grid-wide wait passed, [5] down projection done.  Pass null to switch it off (the default).  Process-wide. */
int ffnk_debug_profile_buffer(void* buffer);

/* Diagnostics: replaces one entry of the compiled-in tile table so that a choice can be timed against its
 * alternatives (`python -m ffn_kernel_b200.tune`; the reference searches its tile configurations offline,
 * find_spec/find.py:18-64).  name: "pair", "narrow", "permute", "epi_warps", "group_m", "wgrad_pair",
 * "max_run_rows", "copy_threshold", "verbose", "route_resident" (0: long masks are routed by the count and
 * scatter kernels even where the one-launch kernel fits), "ksplit" (down projection inside ffnk_ffn_forward: 0 never
 * splits the contraction, n > 1 splits it n ways wherever it can), "early_start" (0: the GEMMs inside
 * ffnk_ffn_forward never start beside their predecessor); value -1 restores the table's own choice.  Process-wide,
 * affects later launches; unknown names return FFNK_ERR_SHAPE.  The library reads no environment variables. */
int ffnk_tune_override(const char* name, int value);

/* Human-readable name of a return code or device status code (static storage). */
const char* ffnk_status_string(int code);

#ifdef __cplusplus
}
#endif
#endif /* FFNK_H_ */
