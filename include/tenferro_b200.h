/*
 * tenferro_b200.h - C ABI of libtenferro_b200.so
 *
 * A B200 (sm_100a) backend for the contraction hot path of tenferro-rs: the
 * `TensorPrims<A>` describe -> plan -> execute protocol and the N-ary einsum
 * contraction-tree executor.  Everything here is plain C: pointers, sizes and
 * integer status codes.  A Rust `CudaBackend: TensorPrims<Standard>` (or any
 * other FFI user) binds exactly these entry points.
 *
 * The reference has no FFI of its own (its C FFI is a stated future goal,
 * AGENTS.md:19-20), so each entry point cites the Rust item whose semantics
 * it carries.
 *
 * Conventions
 *  - Every function returns a tfb_status; TFB_OK is 0.  On failure a
 *    thread-local message is available from tfb_last_error().  Nothing
 *    aborts or throws across this boundary.
 *  - Strides and offsets are signed and counted in ELEMENTS of the dtype,
 *    as in `Tensor<T>` (tenferro-tensor/src/lib.rs:167-171).
 *  - `base` pointers in views are DEVICE pointers.
 *  - Work is enqueued on the context's stream and the call returns without
 *    waiting (tenferro-einsum/src/lib.rs:146-177).  Use events or
 *    tfb_ctx_synchronize() before touching results from the host.
 *  - Complex numbers are interleaved (re, im) pairs.
 */
#ifndef TENFERRO_B200_H
#define TENFERRO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ */
/* Status codes: one per variant of tenferro_device::Error            */
/* (tenferro-device/src/lib.rs:109-159).                              */
/* ------------------------------------------------------------------ */
typedef enum tfb_status {
    TFB_OK = 0,
    TFB_ERR_SHAPE_MISMATCH = 1,       /* Error::ShapeMismatch              */
    TFB_ERR_RANK_MISMATCH = 2,        /* Error::RankMismatch               */
    TFB_ERR_DEVICE = 3,               /* Error::DeviceError(String)        */
    TFB_ERR_NO_COMPATIBLE_DEVICE = 4, /* Error::NoCompatibleComputeDevice  */
    TFB_ERR_CROSS_MEMORY_SPACE = 5,   /* Error::CrossMemorySpaceOperation  */
    TFB_ERR_INVALID_ARGUMENT = 6,     /* Error::InvalidArgument(String)    */
    TFB_ERR_STRIDED = 7               /* Error::Strided(StridedError)      */
} tfb_status;

/* Scalar types with `HasAlgebra<Algebra = Standard>`
 * (tenferro-algebra/src/lib.rs:58-72).  Names follow num-complex:
 * C32 = Complex32 = two f32, C64 = Complex64 = two f64. */
typedef enum tfb_dtype {
    TFB_F32 = 0,
    TFB_F64 = 1,
    TFB_C32 = 2,
    TFB_C64 = 3
} tfb_dtype;

/* PrimDescriptor variants (tenferro-prims/src/lib.rs:152-245). */
typedef enum tfb_op {
    TFB_OP_BATCHED_GEMM = 0,
    TFB_OP_REDUCE = 1,
    TFB_OP_TRACE = 2,
    TFB_OP_PERMUTE = 3,
    TFB_OP_ANTI_TRACE = 4,
    TFB_OP_ANTI_DIAG = 5,
    TFB_OP_CONTRACT = 6,
    TFB_OP_ELEMENTWISE_MUL = 7
} tfb_op;

/* ReduceOp (tenferro-prims/src/lib.rs:100-107). */
typedef enum tfb_reduce_op { TFB_REDUCE_SUM = 0, TFB_REDUCE_MAX = 1, TFB_REDUCE_MIN = 2 } tfb_reduce_op;

/* Extension (tenferro-prims/src/lib.rs:123-128). */
typedef enum tfb_extension { TFB_EXT_CONTRACT = 0, TFB_EXT_ELEMENTWISE_MUL = 1 } tfb_extension;

/* The algebra `TensorPrims<A>` is parameterised by (tenferro-prims/src/lib.rs:278-280): a semiring
 * {zero, one, add, mul} (tenferro-algebra/src/lib.rs:74-106).  Standard is (+, *) on f32, f64,
 * Complex32, Complex64 (:56-72).  MaxPlus (the tropical semiring named at :81-90: add = max,
 * mul = +, zero = -inf, one = 0) and its mirror MinPlus (add = min, zero = +inf) exist for f32
 * and f64. */
typedef enum tfb_algebra { TFB_ALGEBRA_STANDARD = 0, TFB_ALGEBRA_MAX_PLUS = 1, TFB_ALGEBRA_MIN_PLUS = 2 } tfb_algebra;

/* OpKind (tenferro-device/src/lib.rs:77-90). */
typedef enum tfb_op_kind {
    TFB_KIND_CONTRACT = 0,
    TFB_KIND_BATCHED_GEMM = 1,
    TFB_KIND_REDUCE = 2,
    TFB_KIND_TRACE = 3,
    TFB_KIND_PERMUTE = 4,
    TFB_KIND_ELEMENTWISE_MUL = 5
} tfb_op_kind;

/* LogicalMemorySpace (tenferro-device/src/lib.rs:30-38). */
typedef enum tfb_space_kind { TFB_SPACE_MAIN_MEMORY = 0, TFB_SPACE_GPU_MEMORY = 1 } tfb_space_kind;

/* ComputeDevice (tenferro-device/src/lib.rs:46-72). */
typedef enum tfb_device_kind { TFB_DEVICE_CPU = 0, TFB_DEVICE_CUDA = 1, TFB_DEVICE_HIP = 2 } tfb_device_kind;
typedef struct tfb_compute_device {
    int32_t kind;      /* tfb_device_kind */
    int32_t device_id; /* zero-based */
} tfb_compute_device;

/*
 * One PrimDescriptor.  Only the fields of the chosen variant are read:
 *   BATCHED_GEMM   batch_dims[n_batch_dims], m, n, k.  Shapes are
 *                  A[batch..., m, k], B[batch..., k, n], C[batch..., m, n]
 *                  (tenferro-prims/src/lib.rs:156-168).
 *   REDUCE         modes_a, modes_c, reduce_op              (:170-180)
 *   TRACE          modes_a, modes_c, paired[2*n_pairs]      (:182-192)
 *   PERMUTE        modes_a (input), modes_b (output)        (:194-202)
 *   ANTI_TRACE     modes_a, modes_c, paired                 (:204-212)
 *   ANTI_DIAG      modes_a, modes_c, paired                 (:214-222)
 *   CONTRACT       modes_a, modes_b, modes_c                (:227-239)
 *   ELEMENTWISE_MUL  nothing                                (:241-244)
 */
typedef struct tfb_desc {
    int32_t op; /* tfb_op */
    int32_t reduce_op; /* tfb_reduce_op */
    const uint32_t* modes_a;
    size_t n_modes_a;
    const uint32_t* modes_b;
    size_t n_modes_b;
    const uint32_t* modes_c;
    size_t n_modes_c;
    const uint32_t* paired; /* (first, second) label pairs, flattened */
    size_t n_pairs;
    const size_t* batch_dims;
    size_t n_batch_dims;
    size_t m, n, k;
} tfb_desc;

/* View flags. */
#define TFB_VIEW_CONJ 1u /* operand is read as its complex conjugate (lazy Tensor::conj,
                            tenferro-tensor/src/lib.rs:606-658); ignored for real dtypes;
                            not allowed on outputs */

/* A strided device view: the fields of `Tensor<T>` / `StridedView<T>`
 * (tenferro-tensor/src/lib.rs:167-171, 198-211). */
typedef struct tfb_view {
    void* base;               /* device pointer to element 0 of the buffer */
    size_t rank;
    const size_t* dims;       /* [rank] */
    const ptrdiff_t* strides; /* [rank], in elements, may be 0 or negative */
    ptrdiff_t offset;         /* in elements, added to base */
    uint32_t flags;           /* TFB_VIEW_* */
} tfb_view;

typedef struct tfb_ctx tfb_ctx;     /* one per CUDA device in use */
typedef struct tfb_plan tfb_plan;   /* TensorPrims::Plan<T>, immutable after creation */
typedef struct tfb_event tfb_event; /* CompletionEvent */
typedef struct tfb_subscripts tfb_subscripts; /* tenferro_einsum::Subscripts */
typedef struct tfb_tree tfb_tree;   /* tenferro_einsum::ContractionTree */

/* ------------------------------------------------------------------ */
/* Errors                                                              */
/* ------------------------------------------------------------------ */
/* Copy the calling thread's last error message (NUL-terminated) into buf.
 * Returns the full message length. */
size_t tfb_last_error(char* buf, size_t cap);
/* Library version string. */
const char* tfb_version(void);

/* ------------------------------------------------------------------ */
/* tenferro-device: context, stream, stream-ordered pool, events       */
/* ------------------------------------------------------------------ */
/* Create the context of CUDA device `device_id` = ComputeDevice::Cuda{device_id}
 * computing on LogicalMemorySpace::GpuMemory{space_id: device_id}.
 * Fails with TFB_ERR_DEVICE when no usable GPU is present (there is no CPU path). */
tfb_status tfb_ctx_create(int device_id, tfb_ctx** out);
tfb_status tfb_ctx_destroy(tfb_ctx* ctx);
tfb_status tfb_ctx_device(const tfb_ctx* ctx, int* device_id);
/* The CUDA stream (cudaStream_t) all work of this context is enqueued on. */
tfb_status tfb_ctx_stream(const tfb_ctx* ctx, void** stream);
/* Enqueue on a caller-owned stream instead (NULL restores the context's own).  A context is ONE
 * in-order queue: its pool blocks, cached offset tables and split-K scratch are ordered by "the
 * context's stream", so the switch makes the new stream wait for everything already enqueued on
 * the old one.  For work that should overlap (copies beside kernels) use a second context of
 * the same device and chain the two with events. */
tfb_status tfb_ctx_set_stream(tfb_ctx* ctx, void* stream);
tfb_status tfb_ctx_synchronize(tfb_ctx* ctx);
/* Number of SMs and bytes of device memory, as reported by the driver. */
tfb_status tfb_ctx_properties(const tfb_ctx* ctx, int* sm_count, size_t* total_mem, int* cc_major, int* cc_minor);

/* Stream-ordered allocation from the context's own memory pool (created with the context, not
 * the device's default pool): the block is usable by work enqueued after this call and is
 * returned to the pool after work enqueued before tfb_free has finished.  The environment
 * variable TFB_POOL_BYTES, read when the context is created, caps the pool; an allocation
 * past the cap returns TFB_ERR_DEVICE and the context stays usable. */
tfb_status tfb_alloc(tfb_ctx* ctx, size_t bytes, void** out);
tfb_status tfb_free(tfb_ctx* ctx, void* ptr);
/* Bytes currently reserved / in use by the pool. */
tfb_status tfb_pool_stats(tfb_ctx* ctx, size_t* reserved, size_t* used);

tfb_status tfb_memcpy_h2d_async(tfb_ctx* ctx, void* dst, const void* src, size_t bytes);
tfb_status tfb_memcpy_d2h_async(tfb_ctx* ctx, void* dst, const void* src, size_t bytes);
tfb_status tfb_memcpy_d2d_async(tfb_ctx* ctx, void* dst, const void* src, size_t bytes);
/* Pitched copies: `height` rows of `width` bytes, consecutive rows `*_pitch` bytes apart.  This
 * is how a slab of a strided host tensor (a range of one index of a column-major array) travels
 * without a packing pass on the host. */
tfb_status tfb_memcpy_h2d_2d_async(tfb_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                   size_t width, size_t height);
tfb_status tfb_memcpy_d2h_2d_async(tfb_ctx* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                   size_t width, size_t height);
/* GpuMemory{src_device} -> GpuMemory{dst_device} over NVLink
 * (Tensor::to_memory_space_async, tenferro-tensor/src/lib.rs:660-671). */
tfb_status tfb_memcpy_p2p_async(tfb_ctx* ctx, void* dst, int dst_device, const void* src, int src_device, size_t bytes);
tfb_status tfb_memset_async(tfb_ctx* ctx, void* dst, int value, size_t bytes);
/* Page-locked host memory for asynchronous transfers. */
tfb_status tfb_host_alloc(size_t bytes, void** out);
tfb_status tfb_host_free(void* ptr);

/* Measurement support (no counterpart in the reference, which has no benchmarks).
 * tfb_kernel_launch_count: kernels this library has launched in this process.
 * tfb_ctx_profile_begin/read/end: while on, every launch is bracketed by a CUDA event pair on
 * the launching stream; read() waits for the stream and returns the number of launches and
 * the summed device time of the kernel family `kernel` ("contract_dmma", "permute_tiled", ...),
 * each pair's reading less what an empty pair reads (measured by begin()).
 * tfb_probe_*: peak probes - DMMA on register operands (TFLOP/s), streaming copy (GB/s). */
unsigned long long tfb_kernel_launch_count(void);
tfb_status tfb_ctx_profile_begin(tfb_ctx* ctx);
tfb_status tfb_ctx_profile_read(tfb_ctx* ctx, const char* kernel, size_t* launches, double* total_ms);
tfb_status tfb_ctx_profile_end(tfb_ctx* ctx);
tfb_status tfb_probe_fp64_tflops(tfb_ctx* ctx, double* tflops);
tfb_status tfb_probe_hbm_gbs(tfb_ctx* ctx, double* gbs);
/* Dense TF32 rate of tcgen05.mma (128 x 256 x 8 tiles resident in shared memory), TFLOP/s. */
tfb_status tfb_probe_tf32_tflops(tfb_ctx* ctx, double* tflops);
/* The same loop launched back to back for `seconds` (at most 30); reports the rate of the last
 * quarter of the run: what the tensor pipe sustains under the board's power limit. */
tfb_status tfb_probe_tf32_tflops_sustained(tfb_ctx* ctx, double seconds, double* tflops);
/* What one small tcgen05.mma costs: `issuers` threads (1..4, one per warp) of every CTA issue
 * 480 TF32 MMAs of shape m x n x 8 between them (m 64 or 128, n a multiple of 16 up to 256; 128
 * with several issuers), each thread into its own accumulator.  issue_cycles = SM clocks per MMA
 * for the issuing thread, complete_cycles = SM clocks per MMA until all had completed.  The
 * figure behind the grouped kernels' choice of tile and issuer count. */
tfb_status tfb_probe_mma_issue_cycles(tfb_ctx* ctx, int m, int n, int issuers, double* issue_cycles, double* complete_cycles);
/* Self-test of the kernels' bounded waits (no counterpart in the reference): launches one CTA
 * that waits, for at most `polls` polls (1..2^20), on an mbarrier nothing arrives on.  The wait
 * runs out, the kernel records status code 0x7e57 and returns; the next tfb_ctx_synchronize
 * reports TFB_ERR_DEVICE (Error::DeviceError, tenferro-device/src/lib.rs:128-130) with that code
 * in the message and clears it, and the context keeps working. */
tfb_status tfb_selftest_wait_expiry(tfb_ctx* ctx, unsigned polls);

/* Capture and replay of a sequence of calls (no counterpart in the reference, whose executor
 * enqueues node by node; for launch-bound loops such as one site of an MPS sweep).  Between
 * capture_begin and capture_end the calls made on `ctx` enqueue nothing: their
 * launches, pool allocations and copies become the nodes of a graph, which capture_end
 * instantiates.  tfb_graph_launch replays it on the context's stream, with the pointers and
 * scalars the captured calls were given.  The sequence must have run once before it is
 * captured (plans, offset tables and kernel attributes are set up on first use with calls that
 * capture does not allow); synchronize, profile_begin and set_stream are refused while capturing, and
 * events recorded then mark nothing (they read as complete). */
typedef struct tfb_graph tfb_graph;
tfb_status tfb_ctx_capture_begin(tfb_ctx* ctx);
tfb_status tfb_ctx_capture_end(tfb_ctx* ctx, tfb_graph** out);
tfb_status tfb_graph_launch(tfb_graph* graph);
void tfb_graph_destroy(tfb_graph* graph);

/* CompletionEvent (tenferro-tensor/src/lib.rs:301-309, 677-713). */
tfb_status tfb_event_record(tfb_ctx* ctx, tfb_event** out);    /* marks all work enqueued so far */
tfb_status tfb_event_wait(tfb_ctx* ctx, tfb_event* ev);        /* later work of ctx waits for ev; host does not block */
tfb_status tfb_event_synchronize(tfb_event* ev);               /* Tensor::wait */
tfb_status tfb_event_query(tfb_event* ev, int* ready);         /* Tensor::is_ready */
tfb_status tfb_event_elapsed_ms(tfb_event* start, tfb_event* stop, float* ms);
tfb_status tfb_event_destroy(tfb_event* ev);

/* preferred_compute_devices (tenferro-device/src/lib.rs:92-105): devices able to run
 * `op_kind` on the given memory space, most preferred first.  MainMemory has none here
 * (-> TFB_ERR_NO_COMPATIBLE_DEVICE): this library has no CPU path. */
tfb_status tfb_preferred_compute_devices(int32_t space_kind, size_t space_id, int32_t op_kind,
                                         tfb_compute_device* out, size_t cap, size_t* n_out);
/* Display of ComputeDevice: "cpu:0", "cuda:1", "hip:2" (tenferro-device/src/lib.rs:62-72). */
size_t tfb_compute_device_format(tfb_compute_device dev, char* buf, size_t cap);

/* ------------------------------------------------------------------ */
/* tenferro-prims: TensorPrims<Standard> for the CUDA backend          */
/* ------------------------------------------------------------------ */
/* TensorPrims::has_extension_for::<T>(ext) (tenferro-prims/src/lib.rs:322-339). */
int tfb_has_extension(int32_t dtype, int32_t ext);

/* TensorPrims::plan::<T>(desc, shapes) (tenferro-prims/src/lib.rs:282-298).
 * shapes: inputs first, then the output.  Validates the descriptor against the shapes,
 * classifies modes and selects the kernel family.  ctx may be NULL to validate only;
 * such a plan cannot be executed. */
tfb_status tfb_plan_create(tfb_ctx* ctx, const tfb_desc* desc, int32_t dtype, size_t n_shapes,
                           const size_t* ranks, const size_t* const* dims, tfb_plan** out);
tfb_status tfb_plan_destroy(tfb_plan* plan);
/* Name of the kernel family the most recent tfb_execute of this plan used (for logs). */
const char* tfb_plan_kernel_name(const tfb_plan* plan);
/* Pin the contraction kernel family of a plan: 0 automatic (the default), 1 SIMT,
 * 2 FP64 tensor pipe (f64/c64), 3 tcgen05 3xTF32 (f32/c32), 4 FP64 tensor pipe with four real
 * products per complex one.  "Pre-computes kernel selection" (tenferro-prims/src/lib.rs:284-286)
 * made visible so the families can be checked against each other; a forced family that
 * cannot run the layout is an error.
 * About 4: by default a Complex64 product is formed from three real products (Re = P1 - P2,
 * Im = (Ar+Ai)(Br+Bi) - P1 - P2).  The result is exact to a few ulp of its NORM, which is what
 * the 1e-12 relative-Frobenius bound asks; but an imaginary part much smaller than the real part
 * keeps only the digits it shares with it (|Im| = 1e-8 |Re|: about 8 of 16).  Kernel 4, or the
 * environment variable TFB_C64_FOUR_PRODUCTS=1 for every Complex64 product including those of
 * an einsum tree, computes Re and Im each to its own accuracy at roughly 3/4 of the speed. */
tfb_status tfb_plan_force_kernel(tfb_plan* plan, int kernel);

/* `impl TensorPrims<A> for CudaBackend` with A other than Standard: the plan computes over
 * semiring `algebra`,
 *   output = alpha (x) op(inputs) (+) beta (x) output,
 * with every sum of `op` taken with (+) and every product with (x).  For MaxPlus:
 * C[m,n] = max(alpha + max_k(A[m,k] + B[k,n]), beta + C[m,n]); beta = -inf (the semiring's zero)
 * overwrites C without reading it, alpha = 0 (its one) leaves the result as it is.  Tropical
 * plans run on the SIMT kernels (tensor cores only multiply and add); AntiTrace and AntiDiag
 * and the einsum tree executor are Standard-only. */
tfb_status tfb_plan_set_algebra(tfb_plan* plan, int32_t algebra);
/* has_extension_for::<T>(ext) of the backend for algebra A (tenferro-prims/src/lib.rs:322-339). */
int tfb_has_extension_for_algebra(int32_t algebra, int32_t dtype, int32_t ext);

/* TensorPrims::execute (tenferro-prims/src/lib.rs:300-320):
 *   output = alpha * op(inputs) + beta * output
 * alpha and beta point to one host scalar of the plan's dtype.  beta == 0 overwrites
 * the output without reading it.  Views must match the plan's shapes. */
tfb_status tfb_execute(tfb_plan* plan, const void* alpha, size_t n_inputs, const tfb_view* inputs,
                       const void* beta, const tfb_view* output);

/* Reduce without any device allocation.  No counterpart in the reference: it exists for
 * callers that may not allocate on the device at the moment they call - an application
 * whose own allocator owns all device memory, a latency-critical loop, a framework callback
 * where allocation is forbidden.  Same result as a Reduce plan run through tfb_execute:
 *   C[modes_c] = alpha * reduce_op(A[modes_a]) + beta * C[modes_c],  modes_c a subset of modes_a
 * (tenferro-prims/src/lib.rs:170-180 gives the formula), but the partial results of a split
 * reduction are kept in a fixed 4 MiB array inside the library instead of a pool block, and
 * the call uses neither cudaMalloc/cudaFree nor the pool.
 *  - Limit: the output may hold at most 2 MiB (elements x element size); larger outputs are
 *    rejected with TFB_ERR_INVALID_ARGUMENT.  Labels must not repeat inside modes_a.
 *  - The first call on each device looks up the array's device address (one
 *    cudaGetSymbolAddress); make that first call before any stream capture begins.
 *  - All calls share the one array.  Nothing in it needs to start at zero (every slot is
 *    written before it is read), but two calls whose kernels overlap on the GPU - different
 *    streams, different contexts of the same device - race on it; keep them ordered. */
tfb_status tfb_reduce_static(tfb_ctx* ctx, int32_t dtype, int32_t reduce_op, const uint32_t* modes_a, size_t n_modes_a,
                             const tfb_view* a, const uint32_t* modes_c, size_t n_modes_c, const tfb_view* c,
                             const void* alpha, const void* beta);

/* Grouped (ragged) matrix products in one persistent launch:
 *   C_p[m_p, n_p] = alpha * A_p[m_p, k_p] * B_p[k_p, n_p] + beta * C_p   for p in 0..n_problems.
 * `PrimDescriptor::BatchedGemm` covers uniform batches only
 * (tenferro-prims/src/lib.rs:156-168); this entry point carries the same formula to a
 * table of problems with individual sizes.  Strides are in elements. */
typedef struct tfb_gemm_problem {
    int64_t m, n, k;
    const void* a; int64_t a_rs, a_cs; /* A[i,l] at a + i*a_rs + l*a_cs */
    const void* b; int64_t b_rs, b_cs; /* B[l,j] at b + l*b_rs + j*b_cs */
    void* c;       int64_t c_rs, c_cs; /* C[i,j] at c + i*c_rs + j*c_cs */
} tfb_gemm_problem;
/* `problems` is a HOST array; it is copied to the device by this call. */
tfb_status tfb_grouped_gemm(tfb_ctx* ctx, int32_t dtype, size_t n_problems, const tfb_gemm_problem* problems,
                            const void* alpha, const void* beta);
/* The same in the plan/execute form of `TensorPrims` (tenferro-prims/src/lib.rs:284-320): the
 * table is validated, cut into tiles and copied to the device once; every execute is then a
 * single launch with no host-side table work.  The plan keeps the pointers of the table, so
 * the operand buffers must stay where they are while the plan is used. */
typedef struct tfb_grouped_plan tfb_grouped_plan;
tfb_status tfb_grouped_plan_create(tfb_ctx* ctx, int32_t dtype, size_t n_problems, const tfb_gemm_problem* problems,
                                   tfb_grouped_plan** out);
tfb_status tfb_grouped_plan_execute(tfb_grouped_plan* plan, const void* alpha, const void* beta);
void tfb_grouped_plan_destroy(tfb_grouped_plan* plan);

/* ------------------------------------------------------------------ */
/* tenferro-einsum: Subscripts, ContractionTree, executor              */
/* ------------------------------------------------------------------ */
/* Subscripts::new (tenferro-einsum/src/lib.rs:253-258). */
tfb_status tfb_subscripts_new(size_t n_inputs, const size_t* input_ranks, const uint32_t* const* inputs,
                              size_t output_rank, const uint32_t* output, tfb_subscripts** out);
/* Subscripts::parse (tenferro-einsum/src/lib.rs:260-283): "ij,jk->ik"; letters a-z, A-Z;
 * parentheses fix the pairwise order, e.g. "ij,(jk,kl)->il". */
tfb_status tfb_subscripts_parse(const char* notation, tfb_subscripts** out);
tfb_status tfb_subscripts_destroy(tfb_subscripts* subs);
size_t tfb_subscripts_n_inputs(const tfb_subscripts* subs);
size_t tfb_subscripts_input(const tfb_subscripts* subs, size_t i, uint32_t* labels, size_t cap);
size_t tfb_subscripts_output(const tfb_subscripts* subs, uint32_t* labels, size_t cap);
/* 1 when the notation carried parentheses.  The grouping is kept inside the subscripts and
 * honoured by tfb_tree_optimize: each parenthesised group is contracted to one
 * intermediate before it meets its siblings. */
int tfb_subscripts_has_order(const tfb_subscripts* subs);

/* ContractionTree::optimize (tenferro-einsum/src/lib.rs:303-318): minimises the total
 * multiply-add count (exact search for up to 12 operands per group, greedy beyond). */
tfb_status tfb_tree_optimize(const tfb_subscripts* subs, const size_t* ranks, const size_t* const* dims,
                             tfb_tree** out);
/* ContractionTree::from_pairs (tenferro-einsum/src/lib.rs:320-355): intermediates are
 * numbered from n_inputs upward in the order they are produced. */
tfb_status tfb_tree_from_pairs(const tfb_subscripts* subs, const size_t* ranks, const size_t* const* dims,
                               size_t n_pairs, const size_t* pairs, tfb_tree** out);
tfb_status tfb_tree_destroy(tfb_tree* tree);
size_t tfb_tree_n_steps(const tfb_tree* tree);
size_t tfb_tree_pairs(const tfb_tree* tree, size_t* pairs, size_t cap);
/* Multiply-adds of the whole tree (real or complex, whichever the operands are). */
double tfb_tree_macs(const tfb_tree* tree);
size_t tfb_tree_output_dims(const tfb_tree* tree, size_t* dims, size_t cap);

/* einsum_with_plan_into (tenferro-einsum/src/lib.rs:584-621):
 *   output = alpha * einsum(operands) + beta * output
 * walking the tree with every intermediate kept in the context's pool.  The allocating
 * variants (einsum_with_plan, :415-430) are this call on a fresh column-major output
 * with alpha = 1, beta = 0; the `_owned` variants (:482-498) additionally let the
 * caller release operands right after the call returns. */
tfb_status tfb_einsum_with_plan_into(tfb_ctx* ctx, const tfb_tree* tree, int32_t dtype, size_t n_operands,
                                     const tfb_view* operands, const void* alpha, const void* beta,
                                     const tfb_view* output);

#ifdef __cplusplus
}
#endif
#endif /* TENFERRO_B200_H */
