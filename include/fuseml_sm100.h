/*
 * fuseml_sm100.h — C ABI of the sm_100a fused GEMM + epilogue backend.
 *
 * This is the boundary a FuseML maintainer binds in place of the Triton /
 * cuBLAS Lt back half of the reference.  Every entry point takes plain
 * pointers, sizes and strides (no torch types), never allocates or frees
 * device memory, enqueues its work on the CUDA stream it is given and
 * returns without synchronising the host.  Return value: 0 on success, one
 * of the FUSEML_E_* codes otherwise (text via fuseml_sm100_strerror).
 *
 * Reference interfaces replaced (paths inside the FuseML source tree):
 *   - the generated Triton kernel's flat argument list
 *     (fuseml/codegen/kernel_generator.py:695-819, kernel ABI;
 *      fuseml/codegen/kernel_launcher.py:766-814, the launch call)
 *   - aten._addmm_activation / the inline cublasLt addmm_bias_residual
 *     (fuseml/codegen/cublas_epilogue.py:355-571, 602-676)
 *   - the three-tier cost model
 *     (fuseml/passes/topology.py:479-571, fuseml/passes/fusion_pass.py:382-498)
 *   - the SRAM autotuner footprint model
 *     (fuseml/codegen/sram_autotuner.py:135-213)
 */
#ifndef FUSEML_SM100_H_
#define FUSEML_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FUSEML_SM100_ABI_VERSION 3

/* ---- status codes ------------------------------------------------------ */
enum {
  FUSEML_OK = 0,
  FUSEML_E_NULL = 1,          /* a required pointer is null                     */
  FUSEML_E_SHAPE = 2,         /* M, N or K is not positive / exceeds int32      */
  FUSEML_E_DTYPE = 3,         /* dtype combination not supported                */
  FUSEML_E_LAYOUT = 4,        /* stride / alignment not expressible as a TMA map*/
  FUSEML_E_EPILOGUE = 5,      /* unknown opcode, bad operand slot, too many ops */
  FUSEML_E_REDUCTION = 6,     /* bad reduction request                          */
  FUSEML_E_WORKSPACE = 7,     /* workspace missing or too small                 */
  FUSEML_E_PLAN = 8,          /* plan fields out of range                       */
  FUSEML_E_DEVICE = 9,        /* no sm_100 device / driver entry point missing  */
  FUSEML_E_LAUNCH = 10,       /* CUDA reported an error at launch               */
  FUSEML_E_TIMEOUT = 11,      /* a bounded device-side wait ran out             */
  FUSEML_E_LIMIT = 12         /* size beyond a documented fixed maximum         */
};

/* ---- element types ------------------------------------------------------ */
enum {
  FUSEML_BF16 = 0,
  FUSEML_F16 = 1,
  FUSEML_F32 = 2
};

/* ---- epilogue opcodes ---------------------------------------------------
 * The epilogue is a short program run on the fp32 accumulator tile while it
 * is still in registers (the reference emits the same operations as Triton
 * source, fuseml/codegen/kernel_generator.py:1599-1903).  Two value
 * registers exist per element: `acc` and `saved`; SAVE/SWAP/…_SAVED express
 * single-entry DAGs such as gelu(h) * sigmoid(h).
 */
enum {
  FUSEML_OP_NOP = 0,
  FUSEML_OP_RELU = 1,        /* acc = acc > 0 ? acc : 0      (kernel_generator.py:1604) */
  FUSEML_OP_GELU_ERF = 2,    /* 0.5*acc*(1+erf(acc/sqrt2))   (kernel_generator.py:1641) */
  FUSEML_OP_SIGMOID = 3,     /* 1/(1+exp(-acc))              (kernel_generator.py:1655) */
  FUSEML_OP_ADD_IMM = 4,     /* acc += imm                                              */
  FUSEML_OP_MUL_IMM = 5,     /* acc *= imm                                              */
  FUSEML_OP_ADD_T = 6,       /* acc += operand[slot][m,n]  (any stride, 0 = broadcast)  */
  FUSEML_OP_MUL_T = 7,       /* acc *= operand[slot][m,n]                               */
  FUSEML_OP_SAVE = 8,        /* saved = acc                                             */
  FUSEML_OP_SWAP = 9,        /* (acc, saved) = (saved, acc)                             */
  FUSEML_OP_ADD_SAVED = 10,  /* acc += saved                                            */
  FUSEML_OP_MUL_SAVED = 11,  /* acc *= saved                                            */
  FUSEML_OP_GELU_TANH = 12,  /* tanh-approximate GELU (aten.gelu approximate='tanh')    */
  FUSEML_OP_STORE_AUX = 13,  /* aux[slot][m,n] = acc (escape store of an intermediate,  */
                             /*   kernel_generator.py:2020-2039); operand must be       */
                             /*   writable, row-major, same dtype rules as the output   */
  FUSEML_OP_SUB_T = 14,      /* acc -= operand[slot][m,n]                               */
  FUSEML_OP_RSUB_T = 15,     /* acc = operand[slot][m,n] - acc                          */
  FUSEML_OP_GELU_ERF_MUL_SIGMOID = 16, /* acc = gelu_erf(acc) * sigmoid(acc) in one step: the   */
                             /*   diamond SAVE, GELU_ERF, SWAP, SIGMOID, MUL_SAVED (either     */
                             /*   branch order) is rewritten to it at launch when `saved` is   */
                             /*   not read again; half the special-function work              */
  FUSEML_OP_GELU_ERF_BWD_T = 17, /* acc *= gelu'(operand[slot][m,n]), gelu' = Phi(x) + x phi(x):  */
                             /*   aten.gelu_backward(grad = acc, self = operand), the epilogue   */
                             /*   of the data-gradient GEMM of a Linear -> GELU pair            */
  FUSEML_OP__COUNT = 18
};

#define FUSEML_MAX_EPI_OPS 16
#define FUSEML_MAX_OPERANDS 8

typedef struct {
  int32_t opcode;  /* FUSEML_OP_*                              */
  int32_t slot;    /* operand index for *_T / STORE_AUX, else 0 */
  float imm;       /* immediate for *_IMM                       */
  int32_t reserved;
} fuseml_epi_op_t;

/* A 2-D view addressed as ptr[m*stride_m + n*stride_n] (strides in
 * elements; 0 broadcasts that dimension — covers bias[N] (stride_m = 0),
 * per-row vectors (stride_n = 0), expand()ed tensors and full [M,N]
 * residuals (kernel_generator.py:1659-1743). */
typedef struct {
  const void* ptr;
  int64_t stride_m;
  int64_t stride_n;
  int32_t dtype;   /* FUSEML_BF16 | FUSEML_F16 | FUSEML_F32 */
  int32_t reserved;
} fuseml_operand_t;

/* ---- reductions --------------------------------------------------------- */
enum {
  FUSEML_RED_SUM = 1,
  FUSEML_RED_MAX = 2,
  FUSEML_RED_MEAN = 4
};
enum {
  FUSEML_AXIS_N = 1,   /* reduce over columns -> one value per row, out[M]  (dim=-1) */
  FUSEML_AXIS_M = 0,   /* reduce over rows    -> one value per column, out[N] (dim=0) */
  FUSEML_AXIS_ALL = 2  /* reduce over the whole tile grid -> one scalar              */
};

typedef struct {
  int32_t kinds;        /* bit-or of FUSEML_RED_*; 0 = no reduction             */
  int32_t axis;         /* FUSEML_AXIS_*                                        */
  float* out_sum;       /* fp32 outputs, one per requested kind                 */
  float* out_max;
  float* out_mean;
  void* workspace;      /* caller-owned scratch, see fuseml_sm100_workspace_bytes */
  int64_t workspace_bytes;
} fuseml_reduce_t;

/* ---- the GEMM problem --------------------------------------------------- */
typedef struct {
  int64_t M, N, K;
  /* A[M,K]: element (m,k) at a[m*lda + k*a_stride_k] (a_stride_k is the last field of this
   * struct; left at 0 it means 1: K contiguous).                                          */
  const void* a;
  int64_t lda;
  /* B[K,N]: element (k,n) at b[k*b_stride_k + n*b_stride_n]; exactly one of
   * the strides is 1.  b_stride_k == 1 is the nn.Linear weight view
   * (aten.t of W[N,K]); b_stride_n == 1 is a row-major [K,N] matrix.         */
  const void* b;
  int64_t b_stride_k;
  int64_t b_stride_n;
  int32_t ab_dtype;     /* FUSEML_BF16 | FUSEML_F16 | FUSEML_F32 (F32 runs as TF32x3) */
  int32_t out_dtype;    /* dtype of d                                                 */
  /* D[M,N] row-major, leading dimension ldd; may be null when the chain ends
   * in a reduction and the matrix itself is never needed.                    */
  void* d;
  int64_t ldd;
  /* epilogue program                                                         */
  int32_t n_ops;
  int32_t n_operands;
  fuseml_epi_op_t ops[FUSEML_MAX_EPI_OPS];
  fuseml_operand_t operands[FUSEML_MAX_OPERANDS];
  fuseml_reduce_t reduce;
  /* Stride of A along K, in elements: element (m,k) at a[m*lda + k*a_stride_k].  0 or 1: K is
   * contiguous (the usual activation matrix).  Otherwise lda must be 1: A is stored [K,M]
   * (a transposed view, as in a weight gradient dY^T @ X); 16-bit operands then need B row-major
   * [K,N] as well (b_stride_n == 1) and a_stride_k * element size a multiple of 16 bytes. */
  int64_t a_stride_k;
} fuseml_gemm_desc_t;

/* ---- plan: what the roofline router decides ----------------------------- */
/* plan.flags bit: fp32 operands are expanded into the workspace before the MMA (see
 * fuseml_sm100_workspace_bytes).  A caller that launches the same descriptor again with the
 * same workspace and an unchanged B (a weight) may set this bit: the expansion of B found in
 * the workspace is reused and only A is expanded.  The caller vouches that neither B nor that
 * part of the workspace was written in between.                                            */
#define FUSEML_PLAN_B_EXPANSION_VALID 1
/* plan.flags bit: the tiles of a ragged last wave of a CTA-pair launch are shared between all
 * pairs by K ranges; later parts pass through the workspace and are added in a fixed order
 * (fuseml_sm100_schedule shows the walk).  The router sets it when the last wave holds at most
 * half as many tiles as there are CTA pairs (each tile then falls into equal K slices, one per
 * pair) and the K loop is long.  Needs plan.cluster == 2 and plan.grid = 2 x the pairs that run
 * at once; ignored for programs that keep a second value register (SAVE / SWAP / *_SAVED left
 * after the gelu*sigmoid rewrite), which run whole tiles.                                  */
#define FUSEML_PLAN_STREAM_K 2
/* plan.flags bit: group_m counts tile columns, not tile rows: tiles are walked in bands of group_m
 * tile columns (columns fastest inside a band, all tile rows of a band before the next band).
 * The router sets it for long K loops when there are more tile rows than tile columns: a wave
 * of concurrently running tiles is then a compact block of about group_m columns whatever its
 * position, and reads the fewest operand slabs.                                             */
#define FUSEML_PLAN_GROUP_N 4

typedef struct {
  int32_t tile_m;        /* 128                                              */
  int32_t tile_n;        /* 64 | 128 | 256                                   */
  int32_t tile_k;        /* elements per smem stage (128 bytes of K)         */
  int32_t stages;        /* depth of the TMA -> MMA shared-memory ring       */
  int32_t cluster;       /* CTAs cooperating on one MMA (1 or 2)             */
  int32_t acc_stages;    /* TMEM accumulator buffers (epilogue overlap)      */
  int32_t grid;          /* persistent CTAs launched                         */
  int32_t group_m;       /* rasterisation group (tiles along M per sweep)    */
  int32_t smem_bytes;    /* dynamic shared memory requested                  */
  int32_t tmem_cols;     /* TMEM columns allocated per CTA                   */
  int32_t bound;         /* 0 = HBM-bound, 1 = tensor-bound, 2 = latency     */
  int32_t fuse;          /* 1 = run fused kernel, 0 = router declines        */
  int32_t split_k;       /* CTAs sharing one tile's K loop (1 = no split);   */
                         /* > 1: fp32 partial tiles in the workspace, folded */
                         /* and run through the epilogue by a second kernel  */
  int32_t flags;         /* FUSEML_PLAN_* bits, 0 from fuseml_sm100_plan     */
  double flops;          /* 2*M*N*K                                          */
  double bytes;          /* algorithmic HBM bytes                            */
  double t_tensor_us;    /* flops / tensor peak                              */
  double t_hbm_us;       /* bytes / HBM peak                                 */
  double t_est_us;       /* roofline estimate incl. wave quantisation        */
} fuseml_plan_t;

typedef struct {
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  int32_t smem_per_block_optin;   /* bytes */
  int32_t tmem_cols;              /* 512 on sm_100 */
  int32_t l2_bytes;
  double hbm_gbs;                 /* peak used by the router */
  double tensor_tflops;           /* dense bf16 peak used by the router */
} fuseml_device_props_t;

/* Fills props for the current device; with no CUDA device it fills the
 * published B200 figures and returns FUSEML_E_DEVICE.
 * Replaces topology._get_gpu_specs (fuseml/passes/topology.py:386-458). */
int fuseml_sm100_query(fuseml_device_props_t* props);

/* Host-only: choose tile / stage / cluster shape and estimate the run time
 * from a roofline model.  `props` may be null (B200 defaults).
 * Replaces is_compute_bound_gemm (fuseml/passes/topology.py:479-571),
 * _is_tiny_output/_is_compute_bound_trigger (fuseml/passes/fusion_pass.py:382-498)
 * and SRAMAutotuner.get_best_config (fuseml/codegen/sram_autotuner.py:220-447). */
int fuseml_sm100_plan(const fuseml_gemm_desc_t* desc, const fuseml_device_props_t* props,
                      fuseml_plan_t* plan);

/* Bytes of caller-provided scratch the described launch needs (0 when the
 * chain has no reduction and the operands are not fp32). */
int64_t fuseml_sm100_workspace_bytes(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan);

/* Host-only validation of a descriptor (what the launch would check first). */
int fuseml_sm100_validate(const fuseml_gemm_desc_t* desc);

/* D = epilogue(A @ B) and/or its reductions, one fused kernel (+ a small
 * finalize kernel when a reduction is requested).  `plan` may be null.
 * Replaces fused_kernel[grid](...) (fuseml/codegen/kernel_launcher.py:811-814),
 * aten._addmm_activation (fuseml/codegen/cublas_epilogue.py:613-616) and
 * addmm_bias_residual (fuseml/codegen/cublas_epilogue.py:396-557).
 * Stream order: the kernel is launched with programmatic stream serialization and
 * waits on the device for everything enqueued before it on `cuda_stream` before its
 * first global access, so callers order work exactly as for an ordinary launch.
 * The call never allocates, frees or synchronises; work is enqueued only. */
int fuseml_sm100_gemm_epilogue(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan,
                               void* cuda_stream);

/* No counterpart in the reference.  Same contract as fuseml_sm100_gemm_epilogue, for
 * callers that cannot allocate device memory when they launch (code running under
 * another framework's locked memory pool, plugins with a fixed memory budget,
 * allocation-free serving loops): reduction partials and the fp32 operand expansion
 * use a fixed scratch array inside the library instead of desc->reduce.workspace
 * (which is ignored).  The call allocates and frees nothing.
 *   - Limit: the launch may need at most fuseml_sm100_noalloc_scratch_bytes() (8 MiB)
 *     of scratch; more returns FUSEML_E_LIMIT.  Each GPU that loads the library holds
 *     those 8 MiB until the process exits.
 *   - The first call on each device looks up the array's device address; make that
 *     first call before starting any stream capture on that device.
 *   - All calls share the one array: calls that can overlap on the GPU (other
 *     streams, other threads) race on it; keep them on one stream. */
int fuseml_sm100_gemm_epilogue_noalloc(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan,
                                       void* cuda_stream);
int64_t fuseml_sm100_noalloc_scratch_bytes(void);

/* ---- both Linears of a small-M MLP block in one kernel ---------------------
 * y = prog2(prog1(x @ w1^T) @ w2^T) for M <= 128 rows: the intermediate h = prog1(x @ w1^T) is handed
 * from the first GEMM to the second through shared memory and never reaches global memory.  No
 * counterpart in the reference, which runs the two Linears as two kernels with h in HBM between them
 * (benchmarks/bench_mlp_block.py:160-182).  Weights are the nn.Linear tensors as stored:
 * w1[I, D_in], w2[D_out, I], row-major.  prog1 (ops1) runs on h[M, I], prog2 (ops2) on y[M, D_out];
 * both index the shared operand table with their own [m, n].  SAVE / SWAP / *_SAVED and STORE_AUX are
 * not available in ops1.  fp32 runs as 3xTF32.  Work: every CTA takes slices of I, a second pass
 * folds the CTAs' partial outputs in a fixed order (deterministic) and runs prog2.                 */
typedef struct {
  int64_t M, D_in, I, D_out;
  const void* x;   int64_t ldx;    /* x[M, D_in], D_in contiguous                        */
  const void* w1;  int64_t ldw1;   /* w1[I, D_in] row-major                              */
  const void* w2;  int64_t ldw2;   /* w2[D_out, I] row-major                             */
  int32_t ab_dtype, out_dtype;     /* operands (x, w1, w2 share one dtype) and y         */
  void* y;         int64_t ldy;
  int32_t n_ops1, n_ops2, n_operands;
  int32_t flags;                   /* FUSEML_MLP_WEIGHTS_EXPANDED                        */
  fuseml_epi_op_t ops1[FUSEML_MAX_EPI_OPS];
  fuseml_epi_op_t ops2[FUSEML_MAX_EPI_OPS];
  fuseml_operand_t operands[FUSEML_MAX_OPERANDS];
  void* workspace;                 /* fuseml_sm100_mlp_small_workspace_bytes(desc) bytes */
  int64_t workspace_bytes;
} fuseml_mlp_desc_t;

/* fp32 only: the expansions of w1 and w2 found in the workspace are still valid (same contract
 * as FUSEML_PLAN_B_EXPANSION_VALID). */
#define FUSEML_MLP_WEIGHTS_EXPANDED 1

/* Bytes of workspace, or -1 when the block cannot run as one kernel (M > 128, D_out > 512, an I that
 * does not divide into slices of 128 / 64 (16-bit) or 64 / 32 (fp32) columns, rows that are not
 * multiples of 16 bytes, ...): the caller then launches the two Linears separately with
 * fuseml_sm100_gemm_epilogue. */
int64_t fuseml_sm100_mlp_small_workspace_bytes(const fuseml_mlp_desc_t* desc);
int fuseml_sm100_mlp_small(const fuseml_mlp_desc_t* desc, void* cuda_stream);

/* Stand-alone reduction tail over an existing [M,N] matrix (used when the
 * reduction cannot be absorbed into the producing GEMM): sum / max / mean
 * over rows, columns or everything; fp32 results.  Replaces the eager
 * aten.sum/amax/mean tails the reference leaves in the graph when a reduction
 * is not absorbed (fuseml/passes/fusion_pass.py:205-241). */
int fuseml_sm100_reduce_tail(const void* x, int32_t dtype, int64_t M, int64_t N, int64_t ldx,
                             const fuseml_reduce_t* reduce, void* cuda_stream);

/* No counterpart in the reference.  Diagnostics for the bounded device-side waits, applied to
 * every launch made afterwards by this process (0, 0 restores normal operation):
 *   wait_limit_us   wall-clock limit of one wait in microseconds (0 = the built-in 2 s);
 *   drop_last_load  host-injected failure: each CTA's producer issues no TMA load for the last
 *                   K block of its last tile.  The MMA thread then waits on a barrier that nothing
 *                   completes, with no copy in flight, until the limit runs out; the kernel
 *                   records where it gave up, frees its TMEM and returns; the output is undefined
 *                   and fuseml_sm100_device_status reports FUSEML_E_TIMEOUT.
 * Used by the tests of the time-out path; nothing on the GPU faults or traps. */
int fuseml_sm100_set_diagnostics(int64_t wait_limit_us, int32_t drop_last_load);

/* No counterpart in the reference (its Triton grid is one program per tile).  The work one unit
 * (a CTA, or a CTA pair when plan->cluster is 2) of a launch of `desc` under `plan` walks through,
 * in order: whole tiles, and with split-K or FUSEML_PLAN_STREAM_K parts of tiles.  Host
 * arithmetic only, no device needed: the kernel runs the same code.  `*n_units` (may be null)
 * receives the number of units of the launch.  Writes at most `max_items` entries and returns
 * the number of items the unit has (>= 0), or -FUSEML_E_* for a bad descriptor, plan or unit. */
typedef struct {
  int32_t tile;        /* tile index in rasterisation order                                      */
  int32_t kb0, kb1;    /* K blocks [kb0, kb1) of the tile                                         */
  int32_t kind;        /* 0 whole tile; 1 first part, finishes the tile after adding `after`
                          parts from workspace slots slot..slot+after-1; 2 later part, stored to
                          workspace slot `slot`; 3 split-K slice; 4 one K half of a tile two
                          units exchange: stores the columns it does not finish to slot `slot`,
                          adds the partner's part from slot `after` to its own half of the columns
                          (left when kb0 == 0, right otherwise) and finishes that half           */
  int32_t after, slot;
  int32_t tile_m, tile_n; /* the tile's row and column in units of tiles (plan.group_m and
                             FUSEML_PLAN_GROUP_N decide how `tile` maps onto them)                */
} fuseml_work_item_t;
int32_t fuseml_sm100_schedule(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan, int32_t unit,
                              fuseml_work_item_t* items, int32_t max_items, int32_t* n_units);

/* Where a bounded wait gave up (the value fuseml_sm100_device_status returns in *status_out). */
enum {
  FUSEML_WHERE_PRODUCER_EMPTY = 0x201,   /* TMA producer: a ring stage never became free      */
  FUSEML_WHERE_MMA_FULL = 0x202,         /* MMA thread: operands of a K block never arrived   */
  FUSEML_WHERE_MMA_TMEM_EMPTY = 0x203,   /* MMA thread: no accumulator buffer was handed back */
  FUSEML_WHERE_EPILOGUE_TMEM_FULL = 0x204,
  FUSEML_WHERE_PRODUCER_DRAIN = 0x205,
  FUSEML_WHERE_EPILOGUE_TILE_IN = 0x206,
  FUSEML_WHERE_STORE_BOX = 0x207
};

/* Reads and clears the device-side status word written by bounded waits.
 * Synchronises the given stream.  0 = no kernel gave up. */
int fuseml_sm100_device_status(void* cuda_stream, int32_t* status_out);

const char* fuseml_sm100_strerror(int code);
int fuseml_sm100_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FUSEML_SM100_H_ */
