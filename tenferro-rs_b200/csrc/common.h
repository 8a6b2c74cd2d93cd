// Internal declarations shared by the host side and the kernels of libtenferro_b200.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/tenferro_b200.h"

namespace tfb {

// ---------------------------------------------------------------- errors
// Sets the calling thread's message and returns `code`, so call sites read
// `return fail(TFB_ERR_..., "...")`.
tfb_status fail(tfb_status code, const char* fmt, ...);
void set_error(const char* msg);

#define TFB_CUDA(expr)                                                                         \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess)                                                                \
            return ::tfb::fail(TFB_ERR_DEVICE, "%s failed: %s (%s:%d)", #expr,                 \
                               cudaGetErrorString(e__), __FILE__, __LINE__);                   \
    } while (0)

#define TFB_TRY(expr)                    \
    do {                                 \
        tfb_status s__ = (expr);         \
        if (s__ != TFB_OK) return s__;   \
    } while (0)

inline size_t dtype_size(int dt) {
    switch (dt) {
        case TFB_F32: return 4;
        case TFB_F64: return 8;
        case TFB_C32: return 8;
        case TFB_C64: return 16;
    }
    return 0;
}
inline bool dtype_is_complex(int dt) { return dt == TFB_C32 || dt == TFB_C64; }
inline bool dtype_valid(int dt) { return dt >= 0 && dt <= 3; }

// A host scalar of any dtype, widened to complex double.
struct Scalar {
    double re = 0, im = 0;
    bool is_zero() const { return re == 0 && im == 0; }
    bool is_one() const { return re == 1 && im == 0; }
};
Scalar load_scalar(int dtype, const void* p);

}  // namespace tfb

// ---------------------------------------------------------------- context
struct tfb_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;  // own_stream or a caller-provided one
    cudaMemPool_t pool = nullptr;  // the context's own pool (not the device's default one)
    size_t pool_cap = 0;           // TFB_POOL_BYTES at creation, 0: uncapped
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    size_t total_mem = 0;
    size_t smem_optin = 0;
    // One-word device status used by kernels with bounded waits (0 = fine).
    int* dev_status = nullptr;
    // Scratch of the in-kernel stream-K reduction: one accumulator slot and one flag per CTA.
    void* sk_partial = nullptr;
    size_t sk_partial_bytes = 0;
    unsigned* sk_flags = nullptr;
    size_t sk_flags_n = 0;
    unsigned sk_epoch = 0;
    // Optional per-launch timing (tfb_ctx_profile_*): event pairs around named launches.
    bool profiling = false;
    float prof_pair_ms = 0;  // duration an empty event pair reports, subtracted from every launch
    struct ProfRec {
        const char* name;
        cudaEvent_t start, stop;
    };
    std::vector<ProfRec> prof;
    bool capturing = false;  // between tfb_ctx_capture_begin and _end: launches are recorded, not run
};

// A captured sequence of this library's launches, instantiated for replay (tfb_graph_*).
struct tfb_graph {
    tfb_ctx* ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

struct tfb_event {
    cudaEvent_t ev = nullptr;
    int device = 0;
};

namespace tfb {

// Scoped `cudaSetDevice` that restores the caller's device.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// ------------------------------------------------------------ strided ops
constexpr int kMaxRank = 12;  // after fusing adjacent modes

// A loop nest over up to kMaxRank fused modes and up to three tensors.
// Passed to kernels by value.
struct LoopNest {
    int rank = 0;
    int64_t extent[kMaxRank];
    int64_t stride[3][kMaxRank];  // element strides of tensors 0..2 (0 where absent)
    int64_t total = 1;            // product of extents
};

// One mode of a normalised operation: extent and per-tensor element stride.  Tensors 0..2 are
// the operation's own; slot 3 is the fused multiplier of a contraction (0 when there is none).
struct Mode {
    int64_t extent;
    int64_t s[4];
};

// Sort `modes` by |stride| of tensor `key` ascending and fuse neighbours that are
// contiguous in every tensor.  Extent-1 modes vanish.
void sort_and_fuse(std::vector<Mode>& modes, int key, int n_tensors);
// Fuse neighbours only (keeps order).
void fuse_in_order(std::vector<Mode>& modes, int n_tensors);
tfb_status make_nest(const std::vector<Mode>& modes, LoopNest* out);

// Validated view: element pointer already offset, dims/strides as int64.
struct HView {
    char* ptr = nullptr;  // base + offset * sizeof(T)
    std::vector<int64_t> dims, strides;
    bool conj = false;
};
tfb_status to_hview(const tfb_view& v, int dtype, HView* out, const char* what);

// ------------------------------------------------------------ kernel entry points (host launchers)
// out[idx_out] = alpha * (conj?)in[idx_in] + beta * out[idx_out] over nest (tensor 0 = in, 1 = out).
tfb_status launch_permute(tfb_ctx* ctx, int dtype, const LoopNest& nest, const void* in, void* out, Scalar alpha,
                          Scalar beta, bool conj);
// out = alpha * a * b + beta * out (tensors 0,1 = a,b; 2 = out).
tfb_status launch_elementwise_mul(tfb_ctx* ctx, int dtype, const LoopNest& nest, const void* a, const void* b,
                                  void* out, Scalar alpha, Scalar beta, bool conj_a, bool conj_b);
// out[kept] = alpha * reduce_op over `red` of in + beta * out.  kept: tensors (0 = in, 1 = out), red: tensor 0.
tfb_status launch_reduce(tfb_ctx* ctx, int dtype, int op, const LoopNest& kept, const LoopNest& red, const void* in,
                         void* out, Scalar alpha, Scalar beta, bool conj);
// out = beta * out over nest (tensor 0 = out).  beta == 0 writes zeros.
tfb_status launch_scale(tfb_ctx* ctx, int dtype, const LoopNest& nest, void* out, Scalar beta);

// Normalised contraction: C[b,m,n] = alpha * sum_k A[b,m,k] B[b,k,n] + beta * C.
// Each group is a list of fused modes; tensor index 0 = A, 1 = B, 2 = C.
// With `mul` set the sum is multiplied element-wise by D[b,m,n] (tensor index 3, broadcast
// strides allowed) before alpha and beta apply: C = alpha * (A B) . D + beta * C.  This is the
// einsum executor's fusion of a trailing Hadamard node into the product that feeds it.
struct ContractProblem {
    int dtype = TFB_F64;
    std::vector<Mode> batch, m, n, k;
    const void* a = nullptr;
    const void* b = nullptr;
    void* c = nullptr;
    bool conj_a = false, conj_b = false;
    const void* mul = nullptr;
    bool conj_mul = false;
    Scalar alpha, beta;
    int64_t M() const;
    int64_t N() const;
    int64_t K() const;
    int64_t B() const;
};
// The same product with the operands' roles exchanged (C[m,n] = sum_k A B read as
// C[n,m] = sum_k B A): which operand supplies rows and which columns is a matter of names, since
// every mode carries its own strides in A, B and C.  A fused multiplier keeps its strides too.
inline ContractProblem exchange_roles(const ContractProblem& p) {
    ContractProblem q = p;
    std::swap(q.m, q.n);
    std::swap(q.a, q.b);
    std::swap(q.conj_a, q.conj_b);
    for (std::vector<Mode>* grp : {&q.batch, &q.m, &q.n, &q.k})
        for (Mode& md : *grp) std::swap(md.s[0], md.s[1]);
    return q;
}
// CK_DMMA4: the FP64 tensor pipe with FOUR real products per complex one (Complex64 only): slower
// than the default three-product form, but Re and Im are each accurate to their own size.
enum ContractKernel { CK_AUTO = 0, CK_SIMT = 1, CK_DMMA = 2, CK_TCGEN05 = 3, CK_DMMA4 = 4 };
// Runs the problem on ctx's stream.  `used` receives the kernel family chosen.
tfb_status launch_contract(tfb_ctx* ctx, const ContractProblem& p, int force_kernel, const char** used);

// Family-specific launchers (each may decline with *declined = true and TFB_OK).
tfb_status contract_simt(tfb_ctx* ctx, const ContractProblem& p);
// Over a tropical semiring (tfb_algebra: 1 MaxPlus, 2 MinPlus); an empty K group is a single term.
tfb_status contract_simt_semiring(tfb_ctx* ctx, const ContractProblem& p, int algebra);
tfb_status contract_dmma(tfb_ctx* ctx, const ContractProblem& p, bool* declined, bool four_products = false);
tfb_status contract_tcgen05(tfb_ctx* ctx, const ContractProblem& p, bool* declined,
                            const int64_t* const* c_tables = nullptr, const std::vector<Mode>* c_n_modes = nullptr,
                            int c_scale = 1, const std::vector<Mode>* c_m_modes = nullptr,
                            const std::vector<Mode>* c_batch_modes = nullptr);
tfb_status contract_c32_embedded(tfb_ctx* ctx, const ContractProblem& p, bool* declined);

// Scratch from the context pool, released stream-ordered when the object dies.
struct PoolBlock {
    tfb_ctx* ctx = nullptr;
    void* ptr = nullptr;
    ~PoolBlock();
    tfb_status alloc(tfb_ctx* c, size_t bytes);
};

// Device-resident schedule of one problem table for the tensor-core grouped kernels.
struct GroupedFast {
    PoolBlock mem;
    int64_t total_units = 0;
    int grid = 0;
    int pitch = 0;         // tcgen05: records per CTA
    bool tcgen05 = false;  // which kernel the schedule is for
};
tfb_status grouped_tcgen05_prepare(tfb_ctx* ctx, size_t n, const tfb_gemm_problem* problems, GroupedFast* out,
                                   bool* declined);
tfb_status grouped_tcgen05_run(tfb_ctx* ctx, const GroupedFast& f, Scalar alpha, Scalar beta, bool* declined);
tfb_status grouped_tf32_prepare(tfb_ctx* ctx, size_t n, const tfb_gemm_problem* problems, GroupedFast* out,
                                bool* declined);
tfb_status grouped_tf32_run(tfb_ctx* ctx, const GroupedFast& f, Scalar alpha, Scalar beta, bool* declined);
tfb_status grouped_simt(tfb_ctx* ctx, int dtype, size_t n, const tfb_gemm_problem* problems, Scalar alpha, Scalar beta);

int env_int(const char* name, int dflt);

// Counts kernel launches of this library (process-wide) and, while profiling is on, brackets
// the launch with an event pair on the launching stream.
void count_launch(int n = 1);
struct LaunchScope {
    tfb_ctx* ctx;
    cudaEvent_t stop = nullptr;
    LaunchScope(tfb_ctx* c, const char* name);
    ~LaunchScope();
};

}  // namespace tfb
