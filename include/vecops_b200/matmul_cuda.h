/*
 * Thin C ABI over the sm_100a matmul kernels.
 *
 * This is what a vecops build binds in place of its CPU matmul backends.  The
 * semantic is vecops' own (include/vecops/ops/Matmul.h:13-17, :530-570):
 *
 *     C[M,N] = A[M,K] . B[N,K]^T        (B is always addressed as [N,K]; a
 *                                        row-major [K,N] matrix is the view
 *                                        with strides (1, N))
 *
 * with the memory dtype of each operand separate from the compute dtype
 * (docs/Tensor.md:218-231) and an optional per-output-column scale applied in
 * accumulator space before the store conversion
 * (tests/ops/MatmulConversionTestCommon.h:664-671).  The dtype combinations
 * served, and the vecops atoms they stand for (include/vecops/matmul/details/
 * kernel/amx/Atoms.h:51-86):
 *
 *     A      B      C      scale   accumulate   vecops atom
 *     f32    f32    f32    -       f32          (AVX-512 fmadd leaf, amx/Backend.h:767-901): fp32 FMAs on the CUDA cores, or -
 *                                               when the caller brings the scratch the query reports - three tf32 products
 *                                               of split operands on the tensor cores
 *     bf16   bf16   bf16   opt.    f32          AMX_BF16F32 with output<float>(bf16 C)
 *     bf16   bf16   f32    opt.    f32          AMX_BF16F32
 *     f16    f16    f16|f32 opt.   f32          AMX_F16F32 (Atoms.h:74-77), fp16 C through output<float>(fp16 C); same
 *                                               kernels as the bf16 rows (VECOPS_B200_KERNEL_BF16_TCGEN05 or the strided
 *                                               one), the operand format being a field of the instruction descriptor
 *     i8/u8  i8/u8  i32    -       i32 (wraps)  AMX_I8I32<A,B>
 *     bf16   i8     bf16   opt.    f32          AMX_BF16F32 with input<bfloat16_t>(int8 W)
 *     i8/u8  i8/u8  f32|bf16 opt.  i32 (wraps)  AMX_I8I32<A,B> with a dequantising output<int32_t>(float C) transform
 *                                               (tests/ops/MatmulConversionTestCommon.h:501-618): the int32 sum - plus, in
 *                                               the fused form, an int32 accumulator input such as the zero-point
 *                                               correction row - is converted and then scaled / activated
 *
 * All pointers are DEVICE pointers on `device_index`; strides count elements.
 * Nothing here allocates device memory: scratch is passed in by the caller
 * after asking vecops_b200_matmul_workspace (the device counterpart of
 * Matmul::required_workspace, include/vecops/ops/Matmul.h:504-526).  There is
 * no CPU fallback: every entry point that needs a GPU fails with
 * VECOPS_STATUS_EXECUTION_ERROR when none is usable.
 */
#ifndef VECOPS_B200_MATMUL_CUDA_H
#define VECOPS_B200_MATMUL_CUDA_H

#include "vecops_b200/call_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Kernel variants.  AUTO lets the shape/dtype rules decide; the rules are the
 * device counterpart of vecops' runtime_*_profitable predicates
 * (include/vecops/matmul/details/kernel/RuntimeDispatch.h:24-101,
 * src/MatmulRuntimeDispatch.cpp:12-32). */
typedef enum VecopsB200MatmulKernel {
  VECOPS_B200_KERNEL_AUTO = 0,
  VECOPS_B200_KERNEL_GENERIC = 1,      /* strided SIMT; every dtype row above, any shape */
  VECOPS_B200_KERNEL_F32_SIMT = 2,     /* tiled FP32 FMA GEMM */
  VECOPS_B200_KERNEL_BF16_TCGEN05 = 3, /* tcgen05 kind::f16 (bf16 or fp16 operand pairs), TMEM f32 accumulators, TMA pipeline */
  VECOPS_B200_KERNEL_I8_TCGEN05 = 4,   /* tcgen05 kind::i8, TMEM i32 accumulators, TMA pipeline */
  VECOPS_B200_KERNEL_W8_SMALL_M = 5,   /* weight-only int8, M <= 32: 128-bit loads, in-register dequant, split-K */
  VECOPS_B200_KERNEL_W8_TCGEN05 = 6,   /* weight-only int8 on tcgen05: weights widened to bf16 on the way into the dense GEMM's MMAs */
  VECOPS_B200_KERNEL_F32_TF32X3 = 7,   /* FP32 on tcgen05 kind::tf32: both operands split into two tf32 terms, three products summed in fp32
                                          (about 2^-21 relative per product, inside the 1e-5 bar); needs the scratch its query reports */
  VECOPS_B200_KERNEL_COUNT_ = 8
} VecopsB200MatmulKernel;

#define VECOPS_B200_MATMUL_FLAG_ASYNC (1u << 0) /* enqueue only; caller synchronises the stream */

typedef struct VecopsB200Matmul {
  uint32_t struct_size;
  uint32_t kernel;      /* VecopsB200MatmulKernel; AUTO = pick by rules */
  int64_t m, n, k;
  const void* a;        /* [M,K] */
  int64_t a_stride_m, a_stride_k;
  const void* b;        /* [N,K] */
  int64_t b_stride_n, b_stride_k;
  void* c;              /* [M,N] */
  int64_t c_stride_m, c_stride_n;
  const float* column_scale; /* optional [N] f32 factor on the accumulator, NULL = none */
  void* workspace;      /* device scratch, may be NULL when the query returns 0 */
  uint64_t workspace_size;
  void* stream;         /* cudaStream_t; NULL = default stream */
  uint32_t a_dtype, b_dtype, c_dtype; /* VecopsDType */
  int32_t device_index; /* CUDA ordinal; -1 = the calling thread's current device */
  uint32_t flags;
  uint32_t reserved;
} VecopsB200Matmul;

/* Pure host logic, no GPU needed: which kernel the rules choose for this
 * problem (replaces vecops' MatmulRuntimeDispatch for the device path).
 * Fails with INVALID_ARGUMENT on an unsupported dtype row or negative extent,
 * NOT_APPLICABLE when `kernel` was forced to a variant that cannot serve it. */
VECOPS_B200_EXPORT int32_t vecops_b200_matmul_select(const VecopsB200Matmul* problem, uint32_t* kernel,
                                                     VecopsError* error);

/* Bytes of device scratch the chosen kernel needs (split-K partials).  Pure
 * host logic.  Replaces Matmul::required_workspace (ops/Matmul.h:504-526). */
VECOPS_B200_EXPORT int32_t vecops_b200_matmul_workspace(const VecopsB200Matmul* problem, uint64_t* bytes,
                                                        VecopsError* error);

/* Launch.  Synchronous unless VECOPS_B200_MATMUL_FLAG_ASYNC is set.  Replaces
 * Matmul::operator() (ops/Matmul.h:530-570) / kernel::matmul_bound
 * (include/vecops/matmul/details/kernel/Kernel.h:97-133).  M, N or K == 0 are
 * legal: K == 0 stores zeros (ops/Matmul.h:41-43). */
VECOPS_B200_EXPORT int32_t vecops_b200_matmul_run(const VecopsB200Matmul* problem, VecopsError* error);

/* Fused form: COut = convert( activation( (CIn + A . B^T) * alpha * row_scale[m] * column_scale[n] ) ).
 *
 * vecops writes this as the explicit accumulate form `COutput = CInput + A*B^T` (include/vecops/ops/Matmul.h:519-570)
 * with an output transform composed from vec primitives; the compositions its fusion tests use
 * (tests/ops/MatmulFusionTest.cpp:29-120; tests/ops/MatmulConversionTestCommon.h:623-704 runtime and per-column scale,
 * :705-770 bias as a stride-0 CIn + clamp, :1028-1160 relu / sigmoid / silu) are the enumeration below.
 *   - `cin` is optional; its strides count elements and may be 0 (stride_m = 0: a bias row; stride_n = 0: a column).
 *     Float rows take an f32 or bf16 CIn, added in fp32 before anything else.  The int8 row takes an int32 CIn, added
 *     with wraparound ("native integer accumulate"), and nothing else: alpha must be 1 and activation NONE.
 *   - problem->column_scale keeps its meaning and is applied together with alpha.
 *   - Every kernel applies it where it stores C.
 * Workspace and selection are those of the plain problem. */
typedef enum VecopsB200Activation {
  VECOPS_B200_ACTIVATION_NONE = 0,
  VECOPS_B200_ACTIVATION_RELU = 1,
  VECOPS_B200_ACTIVATION_SIGMOID = 2,  /* 1 / (1 + exp(-x)) */
  VECOPS_B200_ACTIVATION_SILU = 3,     /* x / (1 + exp(-x)) */
  VECOPS_B200_ACTIVATION_CLAMP = 4,    /* min(max(x, clamp_lo), clamp_hi) */
  VECOPS_B200_ACTIVATION_COUNT_ = 5
} VecopsB200Activation;

typedef struct VecopsB200Epilogue {
  uint32_t struct_size;
  uint32_t activation;  /* VecopsB200Activation */
  const void* cin;      /* [M,N] accumulator input, NULL = none */
  int64_t cin_stride_m, cin_stride_n;
  uint32_t cin_dtype;   /* VecopsDType: F32 | BF16 (float rows), I32 (int8 row) */
  float alpha;          /* factor on the accumulator, 1 = none */
  float clamp_lo, clamp_hi;
  uint32_t reserved;
  /* Appended (read only when struct_size covers it): an optional f32 factor per OUTPUT ROW, row_scale[m] - with
   * column_scale the row-by-column dequantisation of vecops' per-token quantised matmul, value * row_scales[row] *
   * column_scales[col] (include/vecops/matmul/Quantization.h:195-246; tests/ops/MatmulConversionTestCommon.h:1384-1436).
   * Not for the plain int32 row.  In a batched call over stacked rows the index is the stacked row. */
  const float* row_scale;
} VecopsB200Epilogue;

VECOPS_B200_EXPORT int32_t vecops_b200_matmul_run_fused(const VecopsB200Matmul* problem, const VecopsB200Epilogue* epilogue,
                                                        VecopsError* error);

/* Rank-3 operands: a leading batch axis on A [B,M,K], B [B,N,K] and C [B,M,N], as vecops' operands may carry
 * (tests/ops/MatmulBatchTest.cpp:96-131).  `problem` describes one batch entry; the strides below step from one entry to
 * the next, in elements, and may be 0 for an operand every entry shares (a shared A, or shared weights).
 *   - Shared weights with A and C stacked densely along the batch axis (a_stride_b = M * a_stride_m, likewise C and a
 *     full-matrix CIn) is ONE product with M * count rows: it is run as such.
 *   - Otherwise one launch per entry on problem->stream, asynchronously, and - unless the problem asks for asynchronous
 *     execution - one synchronisation at the end.  Launches share problem->workspace: they are ordered by the stream.
 *   - `epilogue` may be NULL.  cin_stride_b steps its accumulator input (0 = the same bias / matrix for every entry);
 *     column_scale is shared by all entries.
 * Workspace: what vecops_b200_matmul_workspace reports for the problem with m replaced by m * count covers both ways. */
typedef struct VecopsB200Batch {
  uint32_t struct_size;
  uint32_t reserved;
  int64_t count;
  int64_t a_stride_b, b_stride_b, c_stride_b;
  int64_t cin_stride_b;
} VecopsB200Batch;

VECOPS_B200_EXPORT int32_t vecops_b200_matmul_run_batched(const VecopsB200Matmul* problem, const VecopsB200Batch* batch,
                                                          const VecopsB200Epilogue* epilogue, VecopsError* error);

/* The weight-only int8 tensor-core kernel (VECOPS_B200_KERNEL_W8_TCGEN05) with its scratch inside the
 * library instead of in a caller workspace.  It has no counterpart in the reference: it exists for callers
 * of this library that cannot allocate device memory at call time - a serving loop whose memory pool is
 * sealed after start-up, an embedding whose allocator must not be re-entered from an operator, a latency
 * budget that cannot take cudaMalloc's implicit synchronisation.  `workspace` is ignored.
 *
 *   - The scratch is a fixed array of VECOPS_B200_STATIC_SCRATCH_BYTES of device memory that every GPU
 *     holds, from the moment the CUDA runtime loads this library's device code on it (at the latest the
 *     first call of this entry point there) until the process exits.
 *   - Serves bf16 A[M,K] x int8 W[N,K] -> bf16|f32 C, optional column_scale, K % 8 == 0, K-contiguous 16-byte
 *     aligned rows, and as many activation rows as the array has room for: the scratch need (what
 *     vecops_b200_matmul_workspace reports with kernel = W8_TCGEN05) is 81920 * M_pad + 2 * M * K + 5632 bytes,
 *     M_pad = M rounded up to 16, and a problem that needs more than the array holds is refused with
 *     INVALID_ARGUMENT.  That is M <= 80 at K = 4096 and at K = 8192, M <= 96 for any K up to 2048, and never
 *     more than 96 rows.
 *   - Every call on a device shares the array and inherits the previous call's contents (nothing needs
 *     clearing).  Calls that overlap on the GPU - two streams, or asynchronous calls not ordered by one
 *     stream - race on it: serialise them.
 *   - The first call on a device also performs the one-time set-up (device address of the array, kernel
 *     attributes); make that first call before any stream capture begins.
 *   - Calls no cudaMalloc / cudaFree / cudaHostAlloc or any other allocating routine.
 * Synchronous unless VECOPS_B200_MATMUL_FLAG_ASYNC is set; bounded-wait failures are reported by
 * synchronous calls only. */
#define VECOPS_B200_STATIC_SCRATCH_BYTES (8ull << 20)
VECOPS_B200_EXPORT int32_t vecops_b200_matmul_w8_static_scratch(const VecopsB200Matmul* problem, VecopsError* error);

/* Tuning aid: when `device_buffer` (160 x 16 uint64 on the device the kernels run on) is non-NULL the tensor-core
 * kernels write a per-CTA timeline into it (globaltimer stamps and cycle counts of their roles); NULL turns it off.
 * Process-wide; not for concurrent launches. */
VECOPS_B200_EXPORT void vecops_b200_debug_set_trace(void* device_buffer);

/* Stable short name of a variant ("bf16_tcgen05", ...), NULL if out of range. */
VECOPS_B200_EXPORT const char* vecops_b200_kernel_name(uint32_t kernel);

/* Number of usable CUDA devices; 0 when there is no driver or no GPU. */
VECOPS_B200_EXPORT int32_t vecops_b200_device_count(void);

typedef struct VecopsB200DeviceInfo {
  uint32_t struct_size;
  int32_t sm_major, sm_minor;
  int32_t sm_count;
  uint64_t l2_bytes;
  uint64_t hbm_bytes;
  uint64_t smem_per_block_optin;
  char name[64];
} VecopsB200DeviceInfo;

VECOPS_B200_EXPORT int32_t vecops_b200_device_info(int32_t device_index, VecopsB200DeviceInfo* info,
                                                   VecopsError* error);

/* Kernels launched by this library since load (all devices, all threads). */
VECOPS_B200_EXPORT uint64_t vecops_b200_launch_count(void);

/* Waits for everything enqueued on `stream` (a cudaStream_t; NULL = the default stream) - what a caller of the
 * enqueue-only entry points above (quantisers, correction row, pack) does before reading results on the host, without
 * linking the CUDA runtime itself. */
VECOPS_B200_EXPORT int32_t vecops_b200_stream_synchronize(void* stream, VecopsError* error);

/* Device-side wait diagnostics.  Every mbarrier wait in the tensor-core
 * kernels is bounded; a wait that runs out records where it gave up and the
 * kernel returns.  Synchronous runs check this themselves and report
 * EXECUTION_ERROR; after asynchronous runs call this once the stream is
 * idle.  Returns OK and *status == 0 when no wait ever ran out; reading
 * clears the record. */
VECOPS_B200_EXPORT int32_t vecops_b200_take_device_status(int32_t device_index, uint32_t* status,
                                                          VecopsError* error);

/* Column-sharded GEMM with the all-gather of the output fused into the kernel.
 *
 * vecops has no multi-device layer; this is the device form of the N-partition its CPU callers use across
 * threads (one matmul per lane on a sub-view, docs/WorkspacePlanning.md:96-110).  `problem` describes this
 * rank's slab: A[M,K] (replicated), B[n,K] (this rank's rows of B), bf16 in, bf16 or f32 out; problem->c is
 * ignored.  Each finished 32 x 128-byte piece of the slab is TMA-stored from shared memory straight into
 * columns [col0, col0 + n) of EVERY destination in `c` - the full [M, n_total] result of each GPU, own
 * included, reached through peer pointers (CUDA IPC / symmetric memory) - while the main loop continues.
 * Only stores cross GPUs.  The caller orders ranks afterwards (a barrier on the stream) before anyone reads. */
typedef struct VecopsB200Gather {
  uint32_t struct_size;
  int32_t world;       /* number of destinations, 1..8 */
  void* const* c;      /* `world` device pointers: the full C of every rank */
  int64_t n_total;     /* columns of the full C */
  int64_t ldc;         /* row pitch of the full C, elements */
  int64_t col0;        /* first column of this rank's slab */
  uint32_t flags;      /* VECOPS_B200_GATHER_*; a record that ends before this field means 0 */
  uint32_t reserved;
} VecopsB200Gather;

/* c[0] is the NVSwitch MULTICAST address of the result (world must be 1): every finished piece is written once with
 * multimem.st and the switch delivers it into the copy of every GPU bound to the multicast object, the sender's own
 * included - one store leaves the GPU instead of one per peer.  Needs n % 8 == 0 (whole 16-byte stores). */
#define VECOPS_B200_GATHER_MULTICAST (1u << 0)

VECOPS_B200_EXPORT int32_t vecops_b200_matmul_allgather_run(const VecopsB200Matmul* problem, const VecopsB200Gather* gather,
                                                            VecopsError* error);

/* Quantise-on-load, done ahead of the product: dst[m,k] = convert(src[m,k] * scale + zero_point) with vecops' conversion of
 * an fp32 memory element to an 8-bit compute element - truncation toward zero, saturating (quantize_a in
 * tests/ops/MatmulConversionTestCommon.h:549-556).  src f32 or bf16 with element strides; dst u8 or i8, K-contiguous rows. */
VECOPS_B200_EXPORT int32_t vecops_b200_quantize_rows(const void* src, uint32_t src_dtype, int64_t src_stride_m, int64_t src_stride_k,
                                                     void* dst, uint32_t dst_dtype, int64_t dst_stride_m, int64_t rows, int64_t cols,
                                                     float scale, float zero_point, void* stream, VecopsError* error);

/* The same with one multiplier per row in place of `scale`: dst[m,k] = convert(src[m,k] * multipliers[m] + zero_point) - vecops'
 * per-row asymmetric quantisation of the activations (include/vecops/matmul/Quantization.h:76-140,
 * make_runtime_per_row_asymmetric_quantize_transform), whose counterpart on the output side is VecopsB200Epilogue::row_scale. */
VECOPS_B200_EXPORT int32_t vecops_b200_quantize_rows_per_row(const void* src, uint32_t src_dtype, int64_t src_stride_m,
                                                             int64_t src_stride_k, void* dst, uint32_t dst_dtype, int64_t dst_stride_m,
                                                             int64_t rows, int64_t cols, const float* multipliers, float zero_point,
                                                             void* stream, VecopsError* error);

/* out[n] = -zero_point * sum_k B[n,k] for an 8-bit K-contiguous B[N,K]: the int32 accumulator-input row (stride_m = 0) that
 * removes the activations' zero point from an asymmetric product (MatmulConversionTestCommon.h:529-541; the compensation
 * ops::matmul_pack_b_compensated computes, ops/MatmulPack.h:28-35). */
VECOPS_B200_EXPORT int32_t vecops_b200_column_correction(const void* b, uint32_t b_dtype, int64_t b_stride_n, int64_t n, int64_t k,
                                                         int32_t zero_point, int32_t* out, void* stream, VecopsError* error);

/* ---------------------------------------------------------------------------------------------------------------
 * Operand preparation: the device counterpart of ops::matmul_pack (include/vecops/ops/MatmulPack.h:93-131) and of
 * matmul::packed_layout<Atom, Side> (include/vecops/matmul/Packing.h:72-136).
 *
 * vecops packs an operand once into the blocked layout its tile instructions read, and a matmul handed such a tensor
 * skips its own packing stage.  The layout the tensor-core kernels of this library read through TMA is simpler: rows
 * that are K-contiguous, start on 16-byte boundaries and sit on a pitch that is a multiple of 16 bytes.  The packed
 * form is therefore [rows, pitch] with pitch = K rounded up to 128 bytes, elements past K zero - and preparing an
 * operand means bringing any strided view into it: a weight matrix stored [K, N] (C1's layout) is transposed once, an
 * odd K (rows TMA cannot address) gets an aligned pitch, fp32 storage is narrowed to the bf16 / fp16 compute type
 * (the reference's packing converts memory type to compute type too, tests/ops/MatmulPackTest.cpp:339-352).  A matmul
 * "recognises" the packed operand by its strides alone: pass dst as a / b with stride pitch and k-stride 1 and the
 * dispatch picks the tcgen05 kernels where the raw view would have gone to the strided kernel.
 *
 * The same form serves either side (A is [M,K], B is [N,K]); `operand` is recorded for the caller's bookkeeping only.
 */
typedef struct VecopsB200Pack {
  uint32_t struct_size;
  uint32_t operand;          /* 0: A, 1: B */
  int64_t rows, k;           /* logical [rows, K] */
  const void* src;           /* device pointer */
  int64_t src_stride_row, src_stride_k; /* in elements, >= 0 */
  uint32_t src_dtype;        /* VecopsDType */
  uint32_t dst_dtype;        /* same as src_dtype, or bf16 / f16 from an f32 source (round to nearest even) */
  void* dst;                 /* device pointer, 16-byte aligned, not overlapping the source view */
  uint64_t dst_size;         /* bytes available at dst; at least what vecops_b200_matmul_packed_layout reports */
  int32_t device_index;      /* -1: current device */
  uint32_t flags;            /* 0 */
  void* stream;              /* cudaStream_t; the call returns once the kernel is queued */
} VecopsB200Pack;

/* pitch (in elements) and size (bytes) of the packed form of a [rows, K] operand of `dtype`; either output may be NULL. */
VECOPS_B200_EXPORT int32_t vecops_b200_matmul_packed_layout(uint32_t dtype, int64_t rows, int64_t k, int64_t* pitch_elements,
                                                            uint64_t* bytes, VecopsError* error);

/* Fill dst with the packed form of the source view.  rows == 0 or K == 0 touches no memory
 * (tests/ops/MatmulPackTest.cpp:436-459).  INVALID_ARGUMENT for an undersized or unaligned destination, overlap, a
 * dtype pair that is not served. */
VECOPS_B200_EXPORT int32_t vecops_b200_matmul_pack(const VecopsB200Pack* pack, VecopsError* error);

/* ops::matmul_pack_b_compensated (ops/MatmulPack.h:28-35, :104-118): pack a signed 8-bit B and also emit the int32[N]
 * row compensation[n] = -a_zero_point * sum_k B[n,k] - the accumulator input (row stride 0) that removes the zero point
 * of an asymmetrically quantised u8 A from the product.  K == 0 yields an all-zero row. */
VECOPS_B200_EXPORT int32_t vecops_b200_matmul_pack_b_compensated(const VecopsB200Pack* pack, int32_t a_zero_point,
                                                                 int32_t* compensation, VecopsError* error);

/* ---------------------------------------------------------------------------------------------------------------
 * The caller one step above matmul: scaled dot-product attention for one head, composed as vecops composes it
 * (ops::scaled_dot_product_attention, include/vecops/ops/details/attention/SDPA.h:72-84 and :305-383, materialized
 * strategy): S = Q.K^T through the matmul path; s = S*scale + bias, -inf wherever the query mask, the key mask, the
 * keep mask or the causal cut drops the pair (Common.h:200-289); p = softmax row, rounded to the matmul operand type
 * (bf16) - an all-dropped row is all zero (Common.h:293-345); O = P.V through the matmul path again.
 * Q [Lq,Dqk], K [Lkv,Dqk], V [Lkv,Dv] bf16 with element strides, out [Lq,Dv] f32 or bf16.  Masks are bytes (non-zero
 * keeps; the reference takes bool tensors), bias is f32; each may be NULL.  Device scratch (scores, probabilities, the
 * packed V^T and the products' own scratch) is the caller's: ask vecops_b200_sdpa_workspace, pass 256-byte aligned memory.
 * Two strategies, as in the reference (SDPAStrategy, SDPA.h:21-25): `streaming` - one kernel over all heads, the keys walked
 * tile by tile with a running maximum and sum (SparseFlashAttention.h:360-545), nothing of size Lq x Lkv in device memory;
 * it serves bf16 operands with head dims up to 128 and K-contiguous, 16-byte aligned rows of Q and K - and `materialized`
 * (the composition above, any strides).  `automatic` takes streaming whenever it can serve the call; the workspace query
 * and the run make the same choice.  Results of the two differ by the rounding of p (normalised before the bf16 rounding
 * in one, after it in the other), inside the 1e-3 bar of the bf16 rows. */
typedef enum VecopsB200SdpaStrategy {
  VECOPS_B200_SDPA_AUTOMATIC = 0,
  VECOPS_B200_SDPA_MATERIALIZED = 1,
  VECOPS_B200_SDPA_STREAMING = 2 /* NOT_APPLICABLE when the call cannot be served by it */
} VecopsB200SdpaStrategy;

typedef struct VecopsB200Attention {
  uint32_t struct_size;
  uint32_t causal;            /* 0 none, 1 top left (key <= query), 2 bottom right (key <= query + Lkv - Lq) */
  int64_t lq, lkv, dqk, dv;
  const void* q;
  int64_t q_stride_row, q_stride_col;
  const void* k;
  int64_t k_stride_row, k_stride_col;
  const void* v;
  int64_t v_stride_row, v_stride_col;
  void* out;
  int64_t out_stride_row, out_stride_col;
  uint32_t qkv_dtype;         /* VECOPS_DTYPE_BF16 */
  uint32_t out_dtype;         /* F32 | BF16 */
  const uint8_t* query_mask;  /* [Lq] or NULL */
  const uint8_t* key_mask;    /* [Lkv] or NULL */
  const uint8_t* keep_mask;   /* [Lq,Lkv] or NULL */
  int64_t keep_stride_row, keep_stride_col;
  const float* bias;          /* [Lq,Lkv] or NULL, added after the scaling */
  int64_t bias_stride_row, bias_stride_col;
  float scale;
  uint32_t flags;             /* VECOPS_B200_MATMUL_FLAG_ASYNC: enqueue only */
  void* workspace;
  uint64_t workspace_size;
  void* stream;
  int32_t device_index;
  uint32_t strategy;          /* VecopsB200SdpaStrategy; 0 = automatic */
  /* Several heads in one call: head h reads q + h*q_stride_head (elements) and so on; a stride of 0 shares the operand
   * between heads (grouped-query K and V, one mask for all).  heads <= 1 means one head and the strides are ignored.
   * The streaming strategy runs all heads in one launch; the materialized one runs them one after the other on the
   * stream, sharing scratch sized for one head. */
  int64_t heads;
  int64_t q_stride_head, k_stride_head, v_stride_head, out_stride_head;
  int64_t query_mask_stride_head, key_mask_stride_head, keep_stride_head, bias_stride_head;
} VecopsB200Attention;

VECOPS_B200_EXPORT int32_t vecops_b200_sdpa_workspace(const VecopsB200Attention* attention, uint64_t* bytes, VecopsError* error);
VECOPS_B200_EXPORT int32_t vecops_b200_sdpa_run(const VecopsB200Attention* attention, VecopsError* error);
/* Pure host logic: which strategy the run takes for this record (MATERIALIZED or STREAMING) and, for streaming, how many
 * 128-key tiles one work item walks (a query block whose keys span more tiles is cut into chunks that different SMs
 * handle and merge; the cut changes at which running maximum probabilities are rounded to bf16, so a restatement that
 * is to agree beyond 1e-3 needs it).  With workspace_size = 0 the plan is the one the workspace query sized. */
VECOPS_B200_EXPORT int32_t vecops_b200_sdpa_plan(const VecopsB200Attention* attention, uint32_t* strategy, uint32_t* tiles_per_item,
                                                 VecopsError* error);

/* Strided gather of column slabs: dst[M, ldd] columns [col0, col0+cols) <-
 * src[M, cols] (row pitch lds), `elem_size` bytes per element.  Used after the
 * all-gather of a column-sharded GEMM to place peers' slabs into the row-major
 * full matrix. */
VECOPS_B200_EXPORT int32_t vecops_b200_place_columns(void* dst, int64_t ldd, int64_t col0, const void* src,
                                                     int64_t lds, int64_t rows, int64_t cols, uint32_t elem_size,
                                                     void* stream, VecopsError* error);

/* The gather of a column-sharded product as a step of its own, for callers that run it BEHIND the next product
 * (the slab GEMM stores locally at full speed; this call, on a second stream ordered after it by an event, sends the
 * slab while the next GEMM computes).  Columns [col0, col0 + cols) of the local result src[rows, ld] are written to
 * the same columns of every destination in `dst` - the peers' copies of the result, `count` <= 8 pointers this
 * process can store through (symmetric memory, CUDA IPC), visited in the order given (start at the next rank so that
 * no two senders begin on the same receiver).  Only stores cross GPUs.  Asynchronous on `stream`, which belongs to the
 * device `src` lives on - the calling thread's current device; the caller orders the ranks afterwards (a barrier on
 * that stream) before anyone reads.
 *   VECOPS_B200_PUSH_KERNEL       this library's kernel: every 16-byte piece is read once and stored to every destination
 *                                 (16-byte aligned bases, pitch, col0 and cols);
 *   VECOPS_B200_PUSH_COPY_ENGINE  one strided cudaMemcpy2DAsync per destination: no SM is used. */
#define VECOPS_B200_PUSH_KERNEL 0u
#define VECOPS_B200_PUSH_COPY_ENGINE 1u
VECOPS_B200_EXPORT int32_t vecops_b200_push_columns(const void* src, void* const* dst, int32_t count, int64_t ld, int64_t col0,
                                                    int64_t rows, int64_t cols, uint32_t elem_size, uint32_t route, void* stream,
                                                    VecopsError* error);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* VECOPS_B200_MATMUL_CUDA_H */
