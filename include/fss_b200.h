/*
 * fss_b200 -- C ABI of the B200 (sm_100a) sequential-scan library.
 *
 * The library computes the first-order diagonal linear recurrence
 *
 *     h_0 = b_0 ;  h_t = a_t * h_{t-1} + b_t                (forward)
 *     dh_{T-1} = g_{T-1} ;  dh_t = g_t + a_{t+1} * dh_{t+1}
 *     db_t = dh_t ;  da_t = dh_t * h_{t-1} (t>=1) ;  da_0 = 0 (backward)
 *
 * over tensors [B, T, D] (D fastest) of bf16 or fp32 with fp32 state.  It is the native side
 * of the reference project's torch extension `sequential_scan_cuda`
 * (csrc/sequential_scan.cpp:3-23): the four reference functions map to the four functions of
 * the same name below.  Differences from that boundary, on purpose:
 *   - plain C: raw device pointers, sizes, a stream handle in; an int status out
 *     (the reference takes and returns torch::Tensor);
 *   - the caller owns every buffer: outputs and workspace are passed in, nothing is allocated
 *     or freed here (the reference allocates with torch::empty_like, and its bf16 backward
 *     writes grad_beta over the saved forward output, csrc/sequential_scan_kernel.cu:196-197);
 *   - any D >= 1, any T >= 1, 64-bit offsets, row/batch strides, the caller's stream
 *     (the reference accepts five d_model values and launches on the legacy stream,
 *     csrc/sequential_scan_kernel.cu:17-55).
 *
 * All functions return FSS_OK (0) or a negative FSS_E_* code; fss_strerror() names it.  They
 * only enqueue work on `stream`; device-side give-ups (a bounded wait that ran out) are
 * reported through the status word, see fss_scan_ctx.status.
 */
#ifndef FSS_B200_H
#define FSS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FSS_ABI_VERSION 1

/* element types of the [B,T,D] tensors */
#define FSS_DTYPE_BF16 0
#define FSS_DTYPE_F32 1

/* kernel families */
#define FSS_ALGO_AUTO 0     /* single-pass TMA kernel when the layout allows it, else chunked   */
#define FSS_ALGO_CHUNKED 1  /* three launches: chunk summaries, carry composition, chunk re-scan */
#define FSS_ALGO_LOOKBACK 2 /* one persistent launch: TMA tiles + decoupled look-back of carries */

/* return codes */
#define FSS_OK 0
#define FSS_E_NULL (-1)       /* a required pointer is NULL                                  */
#define FSS_E_SHAPE (-2)      /* B, T or D < 0, or a stride smaller than the extent it spans  */
#define FSS_E_DTYPE (-3)      /* dtype is not one of FSS_DTYPE_*                              */
#define FSS_E_WORKSPACE (-4)  /* workspace missing or smaller than fss_workspace_bytes()       */
#define FSS_E_LAYOUT (-5)     /* FSS_ALGO_LOOKBACK asked for a layout it cannot take          */
#define FSS_E_LAUNCH (-6)     /* the CUDA runtime refused a launch (see fss_last_cuda_error)  */
#define FSS_E_ALGO (-7)       /* unknown algorithm id                                         */
#define FSS_E_DEVICE (-8)     /* device query / cudaSetDevice failed                          */
#define FSS_E_TENSORMAP (-9)  /* the driver refused a TMA descriptor                          */
#define FSS_E_ARGS (-10)      /* struct_bytes does not match this header                      */
#define FSS_E_TOO_LARGE (-11) /* problem exceeds a fixed-capacity entry point                 */
#define FSS_E_ALIAS (-12)     /* an output starts at the address of an input / the other output */

/* values the kernels write to the status word (0 = nothing to report) */
#define FSS_STATUS_OK 0
#define FSS_STATUS_LOOKBACK_TIMEOUT 1 /* a tile gave up waiting for its predecessor's carry  */
#define FSS_STATUS_TMA_TIMEOUT 2      /* a tile gave up waiting for its own TMA loads        */
#define FSS_STATUS_EXCHANGE_TIMEOUT 3 /* a rank gave up waiting for another rank's carry     */

/* One [B, T, D] tensor: element (b,t,d) lives at ptr + (b*stride_b + t*stride_t + d) elements. */
typedef struct fss_view {
    void *ptr;
    int64_t stride_b; /* in elements */
    int64_t stride_t; /* in elements; >= D */
} fss_view;

/* What every call needs besides its tensors. */
typedef struct fss_scan_ctx {
    uint32_t struct_bytes; /* sizeof(fss_scan_ctx): guards against header/library skew          */
    int32_t device;        /* CUDA ordinal the buffers live on; -1 = the thread's current device */
    void *stream;          /* cudaStream_t; NULL = legacy default stream                         */
    void *workspace;       /* device scratch, >= fss_workspace_bytes(); zeroed once by           */
    size_t workspace_bytes; /*   fss_workspace_init() and then reused by consecutive launches on
                                ONE stream (two launches sharing it must not overlap)            */
    int32_t *status;       /* device-visible int (device memory or pinned host memory) that a
                              kernel sets to FSS_STATUS_* when it gives up; may be NULL          */
    int32_t algo;          /* FSS_ALGO_*                                                         */
    int32_t flags;         /* FSS_FLAG_*                                                         */
} fss_scan_ctx;

/* Treat the tensors as rows s..s+T-1 of a longer sequence: row 0 DOES read alpha_0 (forward
 * h_0 = a_0*h_in + b_0; the returned product includes a_0) instead of the h_0 = b_0 rule.      */
#define FSS_FLAG_CONTINUATION 1
/* Run-to-run identical results from the single-pass kernels.  By default a tile takes the state
 * that enters it from whichever is published first, its predecessor's final state or a fold of the
 * summaries of several predecessors; the two associate the same sum differently, so the last bits
 * of the fp32 state (rarely one ulp of a bf16 result) depend on timing.  With this flag a tile
 * always waits for its predecessor's final state: one fixed association, bit-identical results in
 * every run, at the price of a serial hand-over per row block (noticeable on long sequences).
 * The chunked kernels are always deterministic.  The reference's kernels are, too: one thread walks
 * a channel group from the first row to the last (csrc/include/sequential_scan_kernel_bf16.cuh:121-151). */
#define FSS_FLAG_DETERMINISTIC 2
/* For the scans.  The single-pass kernels normally release the launch that follows them on the
 * stream at once, so that it can be placed and set itself up while they drain (programmatic
 * dependent launch; the follower still waits for their completion before it touches memory).  With
 * this flag the follower is placed only when the scan has finished.  Measured on B200: the
 * sequence-parallel fix-up kernels, which occupy whole multiprocessors and start with a burst of
 * loads, run 5-9 microseconds faster when they are placed on an empty GPU than when their CTAs were
 * parked one by one behind the scan's last tiles; the local scans of a sequence-parallel step set it. */
#define FSS_FLAG_HOLD_DEPENDENTS 4
/* Test hooks for the bounded waits of the single-pass kernels (no effect on results otherwise):
 * SHORT_WAITS lets every wait give up after a few thousand polls instead of ~a second;
 * MUTE_FIRST_BLOCK makes the tiles of the first row block publish no descriptors, so that the
 * tiles after them wait for something that never arrives, give up, set the status word to
 * FSS_STATUS_LOOKBACK_TIMEOUT and leave (their outputs are then undefined). */
#define FSS_FLAG_TEST_SHORT_WAITS 0x100
#define FSS_FLAG_TEST_MUTE_FIRST_BLOCK 0x200

/* Optional per-column state vectors, all fp32, contiguous [B, D]; any may be NULL.  The single-pass
 * kernels move them as 16-byte words: vectors that are not 16-byte aligned send an FSS_ALGO_AUTO
 * call to the chunked kernels (FSS_ALGO_LOOKBACK: FSS_E_LAYOUT). */
typedef struct fss_forward_state {
    const float *h_in; /* state entering row 0 (needs FSS_FLAG_CONTINUATION); NULL = 0          */
    float *h_last;     /* out: unrounded state after the last row                               */
    float *prod;       /* out: product of alpha over all rows (0 without FSS_FLAG_CONTINUATION) */
    float *block_prod; /* out, [B, nblocks, D]: product of alpha over the rows of block j, for every
                          block j of R = fss_block_rows() rows (rows j*R .. (j+1)*R-1; alpha_0
                          counts as 0 without FSS_FLAG_CONTINUATION); feeds the fix-up         */
    float *block_state; /* out, [B, nblocks, D]: unrounded state after row (j+1)*R-1            */
} fss_forward_state;

typedef struct fss_backward_state {
    const float *u_in;   /* a_T*dh_T arriving from the rows after this tensor; NULL = 0         */
    const float *h_prev; /* h_{-1} for dalpha_0 (needs FSS_FLAG_CONTINUATION); NULL = dalpha_0=0 */
    float *u_out;        /* out: a_0*dh_0, what these rows hand to the rows before them         */
    float *block_prod;   /* out, [B, nblocks, D]: product of alpha over the rows of block j (the same
                            values the forward scan writes); feeds fss_seqpar_fixup_backward      */
    float *block_state;  /* out, [B, nblocks, D]: u = a*dh handed on by row j*R                    */
} fss_backward_state;

/* ---- library information ------------------------------------------------------------- */
int fss_abi_version(void);
const char *fss_strerror(int code);
/* text of the last CUDA runtime error seen by the calling thread in this library */
const char *fss_last_cuda_error(void);

/* ---- workspace ------------------------------------------------------------------------ */
/* Bytes of scratch a forward or backward call on [B,T,D] of `dtype` may use (any algorithm). */
size_t fss_workspace_bytes(int64_t B, int64_t T, int64_t D, int dtype);
/* Zero a freshly allocated workspace (enqueued on `stream`).  Needed once per allocation. */
int fss_workspace_init(void *workspace, size_t bytes, void *stream);

/* ---- the reference's four entry points -------------------------------------------------- */
/* fp32 forward.  Replaces scan_forward (csrc/sequential_scan.cpp:3,13;
 * csrc/sequential_scan_kernel.cu:7-58).  h may not alias alpha or beta. */
int fss_scan_forward(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                     const fss_view *alpha, const fss_view *beta, const fss_view *h);
/* fp32 backward.  Replaces scan_backward (csrc/sequential_scan.cpp:4-6,15;
 * csrc/sequential_scan_kernel.cu:60-124).  h is the saved forward output.
 * In all backward entry points grad_beta may be the very same view as h (same pointer and
 * strides): the gradient then overwrites the saved output, as the reference's bf16 backward
 * does implicitly (csrc/sequential_scan_kernel.cu:197).  Only the look-back algorithm can do
 * this; when the call resolves to FSS_ALGO_CHUNKED it returns FSS_E_LAYOUT and launches
 * nothing.  Any other overlap between the five tensors is not allowed. */
int fss_scan_backward(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                      const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                      const fss_view *grad_alpha, const fss_view *grad_beta);
/* bf16 forward.  Replaces scan_forward_half (csrc/sequential_scan.cpp:8,19;
 * csrc/sequential_scan_kernel.cu:126-187). */
int fss_scan_forward_half(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                          const fss_view *alpha, const fss_view *beta, const fss_view *h);
/* bf16 backward.  Replaces scan_backward_half (csrc/sequential_scan.cpp:9-11,21;
 * csrc/sequential_scan_kernel.cu:189-268).  grad_beta is its own buffer unless the caller
 * passes h's view for it (see fss_scan_backward). */
int fss_scan_backward_half(const fss_scan_ctx *ctx, int64_t B, int64_t T, int64_t D,
                           const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                           const fss_view *grad_alpha, const fss_view *grad_beta);

/* ---- the same scans with explicit dtype and boundary state ------------------------------ */
/* Generalise the four functions above (which call these with state == NULL); the reference has
 * no counterpart for the state vectors -- its kernels always start from h_0 = b_0
 * (csrc/include/sequential_scan_kernel_bf16.cuh:91-100). */
int fss_scan_forward_ex(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                        const fss_view *alpha, const fss_view *beta, const fss_view *h,
                        const fss_forward_state *state);
int fss_scan_backward_ex(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                         const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                         const fss_view *grad_alpha, const fss_view *grad_beta,
                         const fss_backward_state *state);

/* ---- forward scan with the gates of a real-gated linear recurrent unit computed in the kernel ---
 * No counterpart in the reference, whose callers materialise alpha and beta first (the gates are
 * the use case its README.md:3 names).  Per element, with lambda[D] fp32 per channel:
 *     alpha = exp(-8 * softplus(lambda) * sigmoid(r)),  beta = sqrt(1 - alpha^2) * sigmoid(i) * x,
 * both rounded to `dtype` exactly as if they had been stored and re-read, then h = scan(alpha, beta)
 * with the usual first-row rule (h_0 = beta_0 unless FSS_FLAG_CONTINUATION).  Reads r, i, x and
 * writes h: 4 tensor passes instead of the 8 of a gate kernel followed by the scan.
 * bf16 evaluates the gates with the hardware approximations (a and b are rounded to 8 bits
 * anyway), fp32 with the accurate functions.  Single-pass kernel only: layouts it cannot take,
 * and FSS_ALGO_CHUNKED, return FSS_E_LAYOUT; the caller then computes alpha and beta itself.
 * state may carry h_in / h_last; prod, block_prod and block_state must be NULL (FSS_E_ARGS). */
int fss_scan_forward_gated(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                           const fss_view *r, const fss_view *i, const fss_view *x,
                           const float *lambda, const fss_view *h, const fss_forward_state *state);

/* The same gate formulas outside the scan, for the backward of a gated scan (no counterpart in the
 * reference).  fss_gates_forward writes alpha (and beta, unless beta is NULL -- i and x are then
 * unused and may be NULL) exactly as fss_scan_forward_gated forms them internally: the same
 * approximations and the same rounding to `dtype`, so a reverse scan run on this alpha multiplies
 * with bit for bit the values the forward scanned with. */
int fss_gates_forward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                      const fss_view *r, const fss_view *i, const fss_view *x, const float *lambda,
                      const fss_view *alpha, const fss_view *beta);
/* Chain rule through the gates: from the scan's grad_alpha and grad_beta to grad_r, grad_i, grad_x
 * (type `dtype`) and grad_lambda[D] (fp32; ADDED to with atomic operations, so the caller zeroes it
 * first and its last bits depend on the order of the additions).  The derivatives are taken at the
 * unrounded fp32 gate values. */
int fss_gates_backward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                       const fss_view *r, const fss_view *i, const fss_view *x, const float *lambda,
                       const fss_view *grad_alpha, const fss_view *grad_beta, const fss_view *grad_r,
                       const fss_view *grad_i, const fss_view *grad_x, float *grad_lambda);

/* ---- sequence-parallel pieces (no counterpart in the reference, which never splits T) ---- */
/* Rows per block of the block_prod outputs for this problem and algorithm (> 0). */
int64_t fss_block_rows(int dtype, int64_t B, int64_t T, int64_t D, int algo);
/* Fold the gathered per-rank summaries into what enters rank `rank`:
 *   forward : pc = [world][2][B*D] fp32 holding (prod_r, h_last_r) of each rank's zero-state scan;
 *             carry_in[B*D] = state after ranks 0..rank-1.
 *   backward: pc = [world][2][B*D] holding (prod_r, u_out_r); carry_in = u entering from
 *             ranks rank+1..world-1.  One small launch on ctx->stream. */
int fss_seqpar_compose(const fss_scan_ctx *ctx, int backward, int world, int rank, int64_t n,
                       const float *pc, float *carry_in);
/* Carry exchange through peer memory instead of a library all-gather (ranks = GPUs of one box whose
 * memory is mapped into each other's address space, e.g. with CUDA IPC or torch symmetric memory).
 * Rank q owns a table of world*2*n 8-byte cells {fp32 value, 32-bit exchange number} and world+1
 * 32-bit words, all zeroed once before the first exchange (with a barrier between the zeroing and
 * the first push of any rank).  peer_tables / peer_words are HOST arrays of `world` device pointers:
 * entry q is rank q's table / words as mapped in the calling process (entry `rank` is the caller's
 * own, local memory).
 * fss_seqpar_push writes this rank's pair (prod[n], state[n]) as cells into slot `rank` of the
 * tables of the ranks that read it (forward: the later ranks; backward: the earlier ranks -- the
 * others never look at the slot); exchange numbers (`epoch`) start at 1 and grow by one per exchange over the same tables.  A
 * cell that carries the current epoch is complete by itself, so there is no flag and no fence.
 * Before overwriting its slot the push waits until the readers of that slot (forward: later ranks;
 * backward: earlier ranks) have acknowledged exchange epoch-1.
 * fss_seqpar_compose_peer polls the cells of the ranks it folds, composes them like
 * fss_seqpar_compose and acknowledges.  Every wait is bounded; one that runs out sets the status
 * word to FSS_STATUS_EXCHANGE_TIMEOUT and the kernel returns.  world <= 16.  Plain peer stores only:
 * no multicast, no remote loads. */
int fss_seqpar_push(const fss_scan_ctx *ctx, int backward, int world, int rank, int64_t n, const float *prod,
                    const float *state, void *const *peer_tables, void *const *peer_words, uint32_t epoch);
/* The forward push fused with the fold of the per-block products that fss_scan_forward_ex wrote
 * (block_prod [B][nblocks][D], state = h_last [B][D]): computes prod[b][d] = product over the blocks,
 * stores it to prod_out [B][D] and pushes (prod, state) like fss_seqpar_push (forward direction).
 * Needs D % 4 == 0 and 16-byte aligned vectors (else FSS_E_LAYOUT: use fss_scan_forward_ex's prod
 * output and fss_seqpar_push). */
int fss_seqpar_push_blocks(const fss_scan_ctx *ctx, int world, int rank, int64_t B, int64_t nblocks, int64_t D,
                           const float *block_prod, const float *state, float *prod_out,
                           void *const *peer_tables, void *const *peer_words, uint32_t epoch);
int fss_seqpar_compose_peer(const fss_scan_ctx *ctx, int backward, int world, int rank, int64_t n,
                            void *const *peer_tables, void *const *peer_words, uint32_t epoch,
                            float *carry_in);

/* Correct a zero-state forward scan for the state carry_in that really enters row 0: block j is
 * re-scanned from its true entering state
 *     block_state[j-1] + (block_prod[0] * ... * block_prod[j-1]) * carry_in
 * (one rounding per stored value, like the undivided scan) for as long as the second term is not
 * exactly zero for some channel of a group of 32 channel vectors; from the first block where it is
 * zero on, the column already holds the exact result and is left alone.  block_prod, block_state,
 * block_rows are what the zero-state scan wrote.  Needs FSS_FLAG_CONTINUATION. */
int fss_seqpar_fixup_forward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                             const fss_view *alpha, const fss_view *beta, const fss_view *h,
                             const float *carry_in, const float *block_prod, const float *block_state,
                             int64_t block_rows);
/* The same for the backward scan and the u_in that really arrives after the last row: blocks are
 * walked from the last one down and re-scanned from
 *     block_state[j+1] + (block_prod[j+1] * ... * block_prod[nblocks-1]) * u_in
 * while that second term is non-zero.  h_prev is h_{-1} (NULL = 0; used with
 * FSS_FLAG_CONTINUATION, without it row 0 keeps dalpha_0 = 0). */
int fss_seqpar_fixup_backward(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                              const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                              const fss_view *grad_alpha, const fss_view *grad_beta, const float *u_in,
                              const float *h_prev, const float *block_prod, const float *block_state,
                              int64_t block_rows);

/* ---- a forward scan that allocates nothing ------------------------------------------------ */
/* Has no counterpart in the reference.  It exists for callers that cannot obtain scratch memory
 * when they need a scan -- a plugin inside a host that owns all device memory, a loop that must
 * not run into cudaMalloc's device-wide synchronisation, a process whose memory budget is frozen.
 * The chunk summaries of this forward scan (chunked algorithm, h_0 = b_0 rule, no boundary state)
 * go to a fixed array of FSS_NOALLOC_SCRATCH_BYTES that is part of the library image; every GPU
 * that loads the library holds that array until the process exits.  The caller passes only the
 * tensors.  Limits and rules:
 *   - the problem must satisfy  8 * B * D * ceil(T / L) <= FSS_NOALLOC_SCRATCH_BYTES  with L the
 *     chunk length (16..256 rows, chosen like fss_block_rows(..., FSS_ALGO_CHUNKED));
 *     larger problems return FSS_E_TOO_LARGE and launch nothing;
 *   - all calls share the one array: calls whose kernels can overlap on the GPU race and must be
 *     serialised by the caller; nothing in the array needs clearing between calls;
 *   - the first call that targets a device looks up the array's device address; make that first
 *     call before any stream capture starts.
 * No cudaMalloc, cudaFree or other allocating routine is called.  device: CUDA ordinal, or -1 for
 * the calling thread's current device. */
#define FSS_NOALLOC_SCRATCH_BYTES (8u << 20)
int fss_scan_forward_noalloc(int dtype, int device, void *stream, int64_t B, int64_t T, int64_t D,
                             const fss_view *alpha, const fss_view *beta, const fss_view *h);

/* ---- fix-up that folds the exchanged pairs itself ----------------------------------------------
 * The two fix-ups above take a ready-made carry (from fss_seqpar_compose[_peer]).  These variants
 * take the gathered table instead and fold it in their prologue, which saves the composition launch
 * between the exchange and the fix-up:
 *   table       [world][2][B*D] floats in the caller's own memory, filled by a collective (epoch 0);
 *   epoch       0 = `table` is complete when the kernel starts; otherwise the number of the peer
 *               exchange whose cells (in this rank's entry of peer_tables) are polled -- bounded --
 *               and then acknowledged; peer_tables / peer_words are the arrays given to
 *               fss_seqpar_push, `table` is ignored;
 *   carry_out   optional [B*D]: receives the folded carry (the state entering row 0 / the u arriving
 *               after the last row), which the caller needs again (h_prev of the backward);
 *   push_state  optional, peer exchange only (epoch != 0): [B*D], the state THIS rank hands on in the
 *               same exchange.  The fix-up kernel then also does the work of fss_seqpar_push /
 *               fss_seqpar_push_blocks for this rank -- it waits (bounded) until the readers have
 *               acknowledged exchange epoch - 1 and writes the pair into their tables as soon as the
 *               launch before it has finished -- so the caller issues no push for this rank and
 *               exchange.  (A problem whose fix-up grid does not fit on the GPU at once gets the push
 *               as a launch of its own from inside this call; with push_prod NULL that needs D % 4 == 0
 *               and push_prod_out, else FSS_E_LAYOUT.)  With it:
 *   push_prod   [B*D], the product of alpha over this rank's rows; NULL (forward only) = fold
 *               block_prod over the row blocks;
 *   push_prod_out  optional [B*D]: receives that product. */
typedef struct fss_carry_source {
    int32_t world, rank;
    const float *table;
    void *const *peer_tables;
    void *const *peer_words;
    uint32_t epoch;
    float *carry_out;
    const float *push_state;
    const float *push_prod;
    float *push_prod_out;
} fss_carry_source;
int fss_seqpar_fixup_forward_from(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                  const fss_view *alpha, const fss_view *beta, const fss_view *h,
                                  const fss_carry_source *source, const float *block_prod,
                                  const float *block_state, int64_t block_rows);
int fss_seqpar_fixup_backward_from(const fss_scan_ctx *ctx, int dtype, int64_t B, int64_t T, int64_t D,
                                   const fss_view *alpha, const fss_view *h, const fss_view *grad_out,
                                   const fss_view *grad_alpha, const fss_view *grad_beta,
                                   const fss_carry_source *source, const float *h_prev, const float *block_prod,
                                   const float *block_state, int64_t block_rows);

#ifdef __cplusplus
}
#endif
#endif /* FSS_B200_H */
