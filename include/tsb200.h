/*
 * tsb200.h -- C ABI of the B200 (sm_100a) execution library for triton-shared's
 * lowered kernels.
 *
 * What this boundary replaces in the reference
 * --------------------------------------------
 * The reference CPU backend links, per kernel, a generated C++ launcher
 * (backend/driver.py:102-246) against the LLVM-compiled kernel object and calls
 *
 *   extern "C" void <kernel>(int64_t rank, void *memref_desc, ...per pointer...,
 *                            <scalars>..., int nx, int ny, int nz,
 *                            int px, int py, int pz);          (driver.py:109-114)
 *
 * once per program in a serial triple loop (driver.py:116-133).  Inside the
 * kernel every structured load/store is a memref.reinterpret_cast + subview +
 * memref.copy executed by memrefCopy (backend/include/ExecutionEngine/
 * CRunnerUtils.cpp:58-113), and every arithmetic op is a scalar loop.
 *
 * Here the same work is expressed as data: the host side (backend/compiler.py in
 * this package) derives, per memory access, the descriptor that
 * tts.make_tptr/tts.load/tts.store carry (include/triton-shared/Dialect/
 * TritonStructured/IR/TritonStructuredDialect.td:33-121, 300-363) and, per
 * kernel, the op body; the entry points below run a whole range of programs
 * [pid_lo, pid_hi) of the linearised grid as CUDA kernels on a stream.  The
 * library never allocates, frees or owns tensor memory, never synchronises the
 * stream, and reports errors by return code (0 = ok, negative = error; the text
 * is available from tsb_last_error()).  No C++ exception crosses this boundary.
 *
 * Program linearisation: lin = px + nx * (py + ny * pz), the order of the
 * reference's loops flattened with x fastest.  num_programs is always the full
 * grid, also when a caller launches only a sub-range on one of several GPUs.
 */
#ifndef TSB200_H
#define TSB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TSB_MAX_RANK 3
#define TSB_MAX_ACCESSES 24
#define TSB_MAX_OPS 96
#define TSB_NUM_REGS 16
#define TSB_MAX_LOOPS 4

/* element types (what !tt.ptr<T> / tensor<..xT> name) */
enum tsb_dtype {
  TSB_F32 = 0,
  TSB_F16 = 1,
  TSB_BF16 = 2,
  TSB_I32 = 3,
  TSB_I16 = 4,
  TSB_I8 = 5,
  TSB_I1 = 6,  /* stored as one byte, like memref<..xi1> */
  TSB_I64 = 7, /* memory type only: a value is its low 32 bits, sign-extended when stored (index tensors) */
  TSB_F64 = 8,
  TSB_U32 = 9,
  TSB_U16 = 10,
  TSB_U8 = 11
};

enum tsb_error {
  TSB_OK = 0,
  TSB_ERR_INVALID = -1,     /* malformed descriptor / argument */
  TSB_ERR_UNSUPPORTED = -2, /* well-formed but outside what the kernels implement */
  TSB_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed */
  TSB_ERR_TIMEOUT = -4      /* a bounded device-side wait gave up (see tsb_gemm_status) */
};

/*
 * One structured block access of one kernel, evaluated for one launch.
 * Mirrors tts.make_tptr (sizes/strides/offsets) plus the mask dims of
 * tts.load / tts.store (MaskAnalysis.cpp:583-585):
 *
 *   element (i0,..) of the block of program p lives at
 *       base + offset0 + sum_a offset_pid[a]*p[a] + sum_d i_d*strides[d]     (elements)
 *   and is accessed iff for every masked dim d
 *       i_d < dims[d],  dims[d] = max(min(start_d + sizes[d], bound[d]), start_d) - start_d,
 *       start_d = mask_start0[d] + sum_a mask_start_pid[d][a]*p[a]
 *   (StructuredToMemref.cpp:794-853 for loads, 1163-1196 for stores).
 *   A masked load with has_other fills the inaccessible lanes with `other`
 *   (fillWithValue, StructuredToMemref.cpp:192-224); without it those lanes are
 *   unspecified in the reference and read as zero here.
 */
/*
 * Wrap-around (modulo) contribution of one dim to an access's address: the element index gains
 *     scale * ((offset + i_dim * stride) mod modulus),   offset = offset0 + sum_a offset_pid[a]*p[a]
 * which is what `(pid*BLOCK + arange(BLOCK)) % N` scaled by a stride means in the kernel text.
 * The reference lowers the same expression to "split pointers" (two contiguous chunks per
 * block, StructuredToMemref.cpp:263-526); here the modulo is evaluated per lane.
 */
typedef struct tsb_wrap {
  int32_t dim; /* dim of the iteration space */
  int32_t pad_;
  int64_t offset0;
  int64_t offset_pid[3];
  int64_t stride;
  int64_t modulus; /* > 0 */
  int64_t scale;
} tsb_wrap;

typedef struct tsb_access {
  void *base;
  int32_t dtype; /* enum tsb_dtype of the memory element */
  int32_t rank;  /* 1..TSB_MAX_RANK: rank of the iteration space */
  int32_t is_store; /* 0 load, 1 store, 2 mask probe (value 1 where the lane is accessible,
                       no memory read), 3 index probe (value = the lane's linear element
                       offset as i32, no memory read); base may be NULL for 2 and 3 */
  int32_t has_other;
  int64_t offset0;
  int64_t offset_pid[3];
  int64_t sizes[TSB_MAX_RANK];
  int64_t strides[TSB_MAX_RANK]; /* 0 = broadcast along that dim */
  int32_t masked[TSB_MAX_RANK];
  int32_t pad_;
  int64_t mask_start0[TSB_MAX_RANK];
  int64_t mask_start_pid[TSB_MAX_RANK][3];
  int64_t mask_bound[TSB_MAX_RANK];
  uint64_t other_bits; /* bit pattern of `other` in dtype (low bits) */
  int32_t n_wrap;      /* 0..2 wrap-around terms added to the address */
  int32_t pad2_;
  tsb_wrap wrap[2];
  /* per iteration of enclosing loop l (TSB_OP_LOOP_BEGIN slot l) the
   * element offset advances by offset_loop[l] and the mask start of dim d by
   * mask_start_loop[d][l] (loop-carried pointers and `for off in range(0, N, BLOCK)` offsets,
   * PtrAnalysis.cpp:1536-1602).  tsb_elementwise reads them for a loop nest around its body; the other entry points ignore them. */
  int64_t offset_loop[TSB_MAX_LOOPS];
  int64_t mask_start_loop[TSB_MAX_RANK][TSB_MAX_LOOPS];
} tsb_access;

/* Opcodes of the elementwise body (one linalg.generic each in the reference,
 * TritonArithToLinalg.cpp:104; IEEE semantics, no contraction). */
enum tsb_opcode {
  TSB_OP_LOAD = 0,   /* dst <- access[a]                               */
  TSB_OP_STORE = 1,  /* access[a] <- reg b                             */
  TSB_OP_CONST = 2,  /* dst <- imm (bit pattern, type)                 */
  TSB_OP_MOV = 4,
  /* float binary */
  TSB_OP_ADDF = 10, TSB_OP_SUBF, TSB_OP_MULF, TSB_OP_DIVF,
  TSB_OP_MAXNUMF, TSB_OP_MINNUMF, TSB_OP_MAXIMUMF, TSB_OP_MINIMUMF, TSB_OP_REMF,
  /* float unary */
  TSB_OP_EXP = 30, TSB_OP_EXP2, TSB_OP_LOG, TSB_OP_LOG2, TSB_OP_SQRT, TSB_OP_RSQRT,
  TSB_OP_SIN, TSB_OP_COS, TSB_OP_TANH, TSB_OP_ERF, TSB_OP_ABSF, TSB_OP_NEGF,
  TSB_OP_FLOOR, TSB_OP_CEIL,
  /* int binary */
  TSB_OP_ADDI = 50, TSB_OP_SUBI, TSB_OP_MULI, TSB_OP_DIVSI, TSB_OP_REMSI, TSB_OP_DIVUI, TSB_OP_REMUI,
  TSB_OP_MINSI, TSB_OP_MAXSI, TSB_OP_MINUI, TSB_OP_MAXUI,
  TSB_OP_ANDI, TSB_OP_ORI, TSB_OP_XORI, TSB_OP_SHLI, TSB_OP_SHRSI, TSB_OP_SHRUI,
  TSB_OP_ABSI,
  /* compare: imm = predicate (enum tsb_cmp) */
  TSB_OP_CMPF = 80, TSB_OP_CMPI = 81,
  TSB_OP_SELECT = 82, /* dst <- a ? b : c */
  /* casts: imm = source dtype, type = destination dtype */
  TSB_OP_CAST = 90,
  TSB_OP_BITCAST = 91,
  TSB_OP_FMA = 92, /* math.fma: single rounding */
  TSB_OP_REDUCE = 100, /* tsb_block_program: dst <- fold of reg a along dim imm2 with combiner opcode imm;
                          tsb_elementwise: every lane of dst <- fold of reg a over all lanes of the program
                          with combiner opcode imm (blocks of 16 to 4096 lanes, a multiple of 4) */
  TSB_OP_LOOP_BEGIN = 101, /* loop slot a runs imm iterations; tsb_block_program: b = index of the op after its LOOP_END */
  TSB_OP_LOOP_END = 102,   /* closes loop slot a */
  TSB_OP_ARGREDUCE = 103,  /* tsb_block_program only: (dst, c) <- (value, index) of the largest (imm = 1) or smallest
                              (imm = 0) element of reg a along dim imm2, indices from reg b, ties to the smaller index */
  TSB_OP_SCAN = 104        /* tsb_block_program only: dst <- inclusive running combination of reg a along dim imm2 with
                              combiner opcode imm (TSB_OP_ADDF or TSB_OP_ADDI: tl.cumsum, ConversionPatterns.hpp:1941-2007) */
};

enum tsb_cmp {
  /* arith.cmpf */
  TSB_CMPF_OEQ = 1, TSB_CMPF_OGT, TSB_CMPF_OGE, TSB_CMPF_OLT, TSB_CMPF_OLE, TSB_CMPF_ONE, TSB_CMPF_ORD,
  TSB_CMPF_UEQ, TSB_CMPF_UGT, TSB_CMPF_UGE, TSB_CMPF_ULT, TSB_CMPF_ULE, TSB_CMPF_UNE, TSB_CMPF_UNO,
  /* arith.cmpi */
  TSB_CMPI_EQ = 32, TSB_CMPI_NE, TSB_CMPI_SLT, TSB_CMPI_SLE, TSB_CMPI_SGT, TSB_CMPI_SGE,
  TSB_CMPI_ULT, TSB_CMPI_ULE, TSB_CMPI_UGT, TSB_CMPI_UGE
};

/*
 * tsb_elementwise only: besides a register number, an operand (a, b, c, or the b of a store) may be
 *   TSB_REG_ACC  the result of the op executed just before this one (kept in hardware registers), or
 *   TSB_REG_IMM  the 32-bit pattern in imm2 (not for TSB_OP_CAST, which uses imm2 itself);
 * and dst may be TSB_REG_ACC when the only consumer of the result is the next op.  Bodies written
 * with plain register numbers only stay valid.
 */
#define TSB_REG_ACC (-1)
#define TSB_REG_IMM (-2)

/*
 * Data-dependent accesses (gather / scatter, the reference's tts.make_gather_scatter_tptr and
 * unstructured loads/stores, TritonStructuredDialect.td:125-230): a load or store may take a per-lane
 * element index that is added to the access's structured address, and / or a per-lane mask bit that
 * is and-ed with the structured mask.  Flags TSB_MEM_INDEX / TSB_MEM_MASK sit in `imm` for
 * tsb_elementwise bodies and in `imm2` for tsb_block_program bodies (where a store's imm names the
 * dims it walks).  Operands: load  dst <- access[a] (index: b, mask: c);
 *                            store access[a] <- b   (index: c, mask: dst).
 */
#define TSB_MEM_INDEX 1u
#define TSB_MEM_MASK 2u

typedef struct tsb_op {
  int32_t opcode; /* enum tsb_opcode */
  int32_t type;   /* enum tsb_dtype of the result (operand type for compares) */
  int32_t dst, a, b, c; /* register numbers < TSB_NUM_REGS (or TSB_REG_ACC / TSB_REG_IMM), or an access index */
  uint32_t imm;
  uint32_t imm2;
} tsb_op;

/* ------------------------------------------------------------------------- */
/* library state                                                             */

/* Text of the last error on the calling thread ("" if none). */
const char *tsb_last_error(void);
/* Library/ABI version: major*1000 + minor. */
int tsb_version(void);
/* Number of SMs of the current device (used by callers to size partitions). */
int tsb_sm_count(void);

/* ------------------------------------------------------------------------- */
/* generic structured-access engine                                          */

/*
 * Run an elementwise body over programs [pid_lo, pid_hi) of grid[3].
 * Replaces: the reference's per-program call of an LLVM-compiled kernel whose
 * body is {memrefCopy loads, linalg.generic ops, memrefCopy stores}
 * (driver.py:116-133; CRunnerUtils.cpp:58-113; TritonArithToLinalg.cpp:104).
 * All accesses share one iteration space (sizes[] equal); loads of smaller
 * blocks are expressed with stride 0 along broadcast dims.  The body may be wrapped in a perfect
 * loop nest: leading TSB_OP_LOOP_BEGIN ops (a = nesting depth, imm = trip count) matched by
 * trailing TSB_OP_LOOP_END ops; iteration it of depth l shifts every access by offset_loop[l] * it
 * and its mask starts by mask_start_loop[d][l] * it, and the iterations of one program run in order.
 */
int tsb_elementwise(const tsb_access *acc, int n_acc, const tsb_op *ops, int n_ops,
                    const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, void *stream);

/*
 * Run a body that also contains reductions along block axes (tt.reduce) over programs
 * [pid_lo, pid_hi): one CTA per program, every intermediate block held in shared memory.
 * Replaces kernels whose lowered form mixes memref.copy loads/stores, linalg.generic ops and
 * linalg.reduce (ReduceConverter, ConversionPatterns.hpp:1203-1440) without a loop-carried
 * accumulator.  Registers are numbered 0..n_regs-1; reg_masks[r] has bit d set when register r
 * extends along dim d of the iteration space (absent dims are broadcast: a reduction result
 * simply loses the reduced dim).  TSB_OP_STORE carries in imm the mask of dims the store walks.
 * Float reductions combine in a tree, not left to right: results agree with the reference
 * within rounding, not bit for bit.  All block values together must fit 200 KB.
 */
int tsb_block_program(const tsb_access *acc, int n_acc, const tsb_op *ops, int n_ops,
                      const int32_t *reg_masks, int n_regs, const int32_t grid[3], int64_t pid_lo,
                      int64_t pid_hi, void *stream);

/*
 * Plain structured block copy dst[block] <- src[block] for programs
 * [pid_lo,pid_hi): the B200 counterpart of memrefCopy (CRunnerUtils.cpp:58-113)
 * applied to a masked load immediately followed by a masked store.
 */
int tsb_block_copy(const tsb_access *src, const tsb_access *dst, const int32_t grid[3],
                   int64_t pid_lo, int64_t pid_hi, void *stream);

/* ------------------------------------------------------------------------- */
/* row kernels (one program per row)                                         */

/*
 * Fused row softmax for rows [row_lo,row_hi): per row r
 *   x = load(in + r*in_row_stride + [0,block), mask < n_cols, other=-inf)
 *   y = exp(x - max(x)) / sum(exp(x - max(x)));  store(out + r*out_row_stride, mask)
 * Replaces the lowered form pinned by test/Conversion/StructuredToMemref/
 * kernel-02-fused-softmax.mlir:50-90 (fill -inf, subview copy, linalg.reduce
 * maxnumf, linalg.generic subf/exp, linalg.reduce addf, divf, masked store).
 * dtype: TSB_F32, TSB_F16 or TSB_BF16 in memory; arithmetic is fp32 for f32 input.
 */
int tsb_softmax_rows(const void *in, void *out, int32_t dtype, int64_t in_row_stride,
                     int64_t out_row_stride, int64_t n_cols, int64_t block, int64_t row_lo,
                     int64_t row_hi, void *stream);

/*
 * LayerNorm forward for rows [row_lo,row_hi) (the kernel of
 * python/examples/test_layernorm.py:29-76, lowered form pinned by
 * test/Conversion/StructuredToMemref/kernel-05-layer-norm-fwd.mlir):
 *   mean = sum(x)/N; var = sum((x-mean)^2)/N; rstd = 1/sqrt(var+eps)
 *   y = ((x-mean)*rstd)*w + b, rounded to the I/O dtype; mean,rstd stored fp32.
 * x,y,w,b share io_dtype (TSB_F16, TSB_BF16 or TSB_F32); math is fp32.
 * mean/rstd may be NULL (then not stored).
 */
int tsb_layernorm_fwd(const void *x, void *y, const void *w, const void *b, float *mean,
                      float *rstd, int32_t io_dtype, int64_t x_row_stride, int64_t y_row_stride,
                      int64_t n_cols, float eps, int64_t row_lo, int64_t row_hi, void *stream);

/* ------------------------------------------------------------------------- */
/* reductions                                                                */

/*
 * Strided masked 2-D sum along axis 1:
 *   out[i*out_stride] = sum_{j < n_valid} x[i*stride_m + j*stride_n],  row_lo <= i < row_hi
 * fp32 in, fp32 accumulate.  Either stride may be the unit one: stride_m == 1
 * (the kept dim is memory-contiguous, "column sums of a row-major matrix") or
 * stride_n == 1 (plain row sums).  Replaces a loop of masked 2-D block loads
 * (test/Conversion/StructuredToMemref/masked_ldst_2d.mlir:76-99) each followed by
 * linalg.reduce addf over axis 1 (reducesum_512_256_f32_axis1.mlir) and an addf
 * into the running row sums.
 *
 * `scratch` is caller-provided device memory of at least
 * tsb_reduce_rows_scratch_bytes(row_hi-row_lo, n_valid, stride_m, stride_n) bytes
 * holding per-split partial sums; it may be NULL when that size is 0.  With stride_m == 1 and
 * enough rows to fill the GPU with at most 16 column splits per 128-row tile the splits are
 * combined inside a thread-block cluster (one launch, no scratch); matrices of few rows and
 * very many columns use the scratch partial sums and a second, combining launch.
 */
int64_t tsb_reduce_rows_scratch_bytes(int64_t n_rows, int64_t n_valid, int64_t stride_m,
                                      int64_t stride_n);
int tsb_reduce_rows(const float *x, float *out, int64_t stride_m, int64_t stride_n,
                    int64_t out_stride, int64_t n_valid, int64_t row_lo, int64_t row_hi,
                    void *scratch, void *stream);

/*
 * tsb_reduce_rows for hosts that cannot allocate device memory (no counterpart in the
 * reference, which never allocates on a device).  Meant for launchers without an
 * allocator of their own (plain C / ctypes), for processes whose device memory is
 * entirely managed by another framework's arena, and for latency-critical loops that
 * must avoid the device-wide synchronisation cudaMalloc and cudaFree can cause.
 * The per-split partial sums go to a fixed array in the library's device image:
 * TSB_REDUCE_STATIC_SCRATCH_BYTES per GPU, resident from library load to process exit.
 * A shape whose partials need more (see tsb_reduce_rows_scratch_bytes) is refused
 * with TSB_ERR_UNSUPPORTED.  Same arguments and results as tsb_reduce_rows.
 * All calls on one device share the array: calls that overlap on the GPU race, so
 * keep them on one stream or order them with events.  The first call on a device
 * looks the array's address up and should precede any stream capture.
 */
#define TSB_REDUCE_STATIC_SCRATCH_BYTES (1u << 20)
int tsb_reduce_rows_static(const float *x, float *out, int64_t stride_m, int64_t stride_n,
                           int64_t out_stride, int64_t n_valid, int64_t row_lo, int64_t row_hi,
                           void *stream);

/*
 * Full sum of n fp32 values x[i*stride] into out[0] (one program, 1-D block
 * loads + linalg.reduce addf into a rank-0 tensor, reducesum_scalar.mlir:21-31).
 * Deterministic: fixed tree order for given n.
 */
int tsb_reduce_all(const float *x, float *out, int64_t n, int64_t stride, void *stream);

/* ------------------------------------------------------------------------- */
/* tt.dot path                                                               */

/*
 * Blocked matmul C[M,N] = A[M,K] * B[K,N] for the output tiles owned by programs
 * [pid_lo,pid_hi): fp32 accumulation over ascending K, one rounding to the
 * output type (MatmulConverter, ConversionPatterns.hpp:1128-1201; lowered loop
 * test/Conversion/StructuredToMemref/kernel-03-matrix-multiplication.mlir:157-204).
 * A, B, C are TSB_BF16 or TSB_F16 (same type). Strides in elements.  The unit
 * stride of A must be K (stride_ak == 1); B may be [K,N] row-major
 * (stride_bn == 1) or column-major (stride_bk == 1); stride_cn == 1.
 * tile_of_pid: device array of int32 pairs (tile_m, tile_n) for every program of
 * the FULL grid (n_programs entries), i.e. the kernel's own pid -> tile mapping
 * (grouped swizzle, test_matmul.py:57-65) evaluated by the host.
 * block_m/n/k: the kernel's BLOCK sizes; block_m must be 128, block_n a
 * multiple of 16 in [16,256], block_k a multiple of 64.
 * status: device int32[4]; status[0] != 0 after completion means a bounded wait
 * inside the kernel gave up (the output is then invalid). May be NULL.
 */
int tsb_gemm(const void *a, const void *b, void *c, int32_t dtype, int64_t M, int64_t N, int64_t K,
             int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
             int64_t stride_cm, int64_t stride_cn, int32_t block_m, int32_t block_n,
             int32_t block_k, const int32_t *tile_of_pid, int64_t n_programs, int64_t pid_lo,
             int64_t pid_hi, int32_t *status, void *stream);

/*
 * Same product as tsb_gemm for PAIRS of vertically adjacent tiles: entry w of `pairs` (device
 * int32 pairs) names tiles (tile_m, tile_n) and (tile_m + 1, tile_n), which two CTAs on two SMs
 * compute together with tcgen05.mma.cta_group::2; each CTA stages its own A rows and half of the
 * B block, which cuts shared-memory traffic per SM by a third.  Replaces the same reference loop
 * nest as tsb_gemm (kernel-03-matrix-multiplication.mlir:157-204).  Requires block_m == 128,
 * K > 0 and operands eligible for the tensor path (16-byte aligned bases and row pitches,
 * unit stride along K for A, along N or K for B, block_n a multiple of 128 for [K,N] B and of
 * 32 for [N,K] B); otherwise TSB_ERR_UNSUPPORTED is returned and nothing is launched, and the
 * caller uses tsb_gemm.  A tile_m + 1 beyond M is allowed (its rows are never stored).
 */
int tsb_gemm_paired(const void *a, const void *b, void *c, int32_t dtype, int64_t M, int64_t N, int64_t K,
                    int64_t stride_am, int64_t stride_ak, int64_t stride_bk, int64_t stride_bn,
                    int64_t stride_cm, int64_t stride_cn, int32_t block_m, int32_t block_n,
                    int32_t block_k, const int32_t *pairs, int64_t n_pairs, int32_t *status,
                    void *stream);

/* ------------------------------------------------------------------------- */
/* launch plans                                                              */

/*
 * A launch plan is the JSON text that this package's Triton backend emits as a kernel's "binary"
 * (stage `plan`; it is also what TRITON_SHARED_DUMP_PATH/plan.json holds): a kernel family and its
 * parameters as polynomials over the kernel's integer arguments, program ids and grid sizes.
 * tsb_plan_create parses it once; tsb_launch evaluates it for one call and launches programs
 * [pid_lo, pid_hi) of grid[3] on `stream`.  Replaces what the reference's generated launcher does
 * after unmarshalling its arguments (backend/driver.py:102-246): the serial loop over the compiled
 * kernel.  Arguments are indexed by position in the kernel's signature without its constexpr
 * parameters: ptr_args[i] is the device address of pointer argument i (ignored elsewhere),
 * scalar_args[i] the value of scalar argument i (kind TSB_SCALAR_NONE for pointers).
 *
 * The library allocates no device memory: a launch that needs device scratch (partial sums of a
 * reduction, the pid -> tile table of a matmul) takes it from `scratch`, at least
 * tsb_launch_scratch_bytes(...) bytes for the same plan, grid, range and scalars (0 = none needed);
 * launches that share scratch must be ordered on one stream.  `status` is the int32[4] word of
 * tsb_gemm (may be NULL).  A plan handle may be used from several threads.
 * tsb_plan_create returns NULL on error; the other calls return 0 or a negative tsb_error.
 */
typedef struct tsb_plan tsb_plan;
enum tsb_scalar_kind { TSB_SCALAR_NONE = 0, TSB_SCALAR_INT = 1, TSB_SCALAR_FLOAT = 2 };
typedef struct tsb_scalar {
  int32_t kind; /* enum tsb_scalar_kind */
  int32_t pad_;
  int64_t i;    /* value of an integer argument (i1 ... i64, u8 ... u64) */
  double f;     /* value of a floating-point argument (fp32, fp64) */
} tsb_scalar;

tsb_plan *tsb_plan_create(const char *json, int64_t length /* < 0: NUL-terminated */);
void tsb_plan_destroy(tsb_plan *plan);
const char *tsb_plan_family(const tsb_plan *plan);
const char *tsb_plan_kernel_name(const tsb_plan *plan);
int64_t tsb_launch_scratch_bytes(const tsb_plan *plan, const int32_t grid[3], int64_t pid_lo, int64_t pid_hi,
                                 const tsb_scalar *scalar_args, int n_args);
int tsb_launch(const tsb_plan *plan, const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, void *stream,
               void *const *ptr_args, const tsb_scalar *scalar_args, int n_args, void *scratch,
               int64_t scratch_bytes, int32_t *status);

#ifdef __cplusplus
}
#endif
#endif /* TSB200_H */
