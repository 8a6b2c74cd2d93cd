// Peak probes for the roofline denominators that no library call measures: the FP64 tensor
// pipe (DMMA) on register-resident operands, and a plain streaming copy for HBM.
#include "common.h"
#include "ptx_sm100.cuh"

namespace tfb {

// Each warp keeps 8 independent m8n8k4 accumulators busy; nothing touches memory in the loop.
__global__ void __launch_bounds__(256) probe_dmma_kernel(double* sink, int iters, double seed) {
    double c[8][2];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i][0] = c[i][1] = 0.0;
    double a = seed + threadIdx.x * 1e-9, b = seed * 0.5 + threadIdx.x * 1e-9;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                         : "+d"(c[i][0]), "+d"(c[i][1])
                         : "d"(a), "d"(b));
    }
    double s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += c[i][0] + c[i][1];
    if (s == 12345.678) sink[0] = s;  // keeps the loop alive without a store in practice
}

__global__ void __launch_bounds__(256) probe_copy_kernel(const uint4* __restrict__ in, uint4* out, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = in[i];
}

// Self-test of the bounded wait every kernel here relies on: one CTA sets up an mbarrier that
// nothing ever arrives on, waits for it with a small poll limit, and returns.  The wait must
// run out, leave its code in the status word and let the kernel end normally.
constexpr int kSelftestWaitCode = 0x7e57;
__global__ void __launch_bounds__(32) selftest_wait_expiry_kernel(int* status, unsigned polls, unsigned* polls_done) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (threadIdx.x == 0) {
        mbar_wait(b, 0, status, kSelftestWaitCode, polls);
        if (polls_done) *polls_done = polls;
    }
}

// What one tcgen05.mma costs the thread that issues it.  `issuers` threads (one per warp) of a CTA
// each issue `per_issuer` TF32 MMAs of shape m x n x 8 on operands that sit in shared memory, each
// thread into its own accumulator, then commit and wait.  out[0] = clocks until the slowest
// issuer had issued its share, out[1] = clocks until all MMAs had completed.
__global__ void __launch_bounds__(128, 1) probe_mma_issue_kernel(int issuers, int per_issuer, int m, int n, long long* out,
                                                                 int* status) {
    extern __shared__ char smem_raw[];
    char* smem = (char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t base = smem_u32(smem);
    const uint32_t bars = base + 64 * 1024;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 16 * 1024; i += 128) ((float*)smem)[i] = 1.0f;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(bars + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(bars + 64, 512);
        tmem_relinquish();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)(smem + 64 * 1024 + 64);
    __shared__ long long t_issue[4], t_done[4];
    if (lane == 0 && warp < issuers) {
        // A: MN-major boxes of [32 k][32 m], B: K-major rows of 128 bytes (the layouts of the grouped kernel)
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
        const uint64_t hi = (1ull << 46);
        const uint64_t da = (uint64_t)((base & 0x3FFFFu) >> 4) | ((uint64_t)(4096u >> 4) << 16) | ((uint64_t)(512u >> 4) << 32) | hi | (1ull << 61);
        const uint64_t db = (uint64_t)(((base + 32768u) & 0x3FFFFu) >> 4) | ((uint64_t)(16u >> 4) << 16) | ((uint64_t)(1024u >> 4) << 32) | hi | (2ull << 61);
        const uint32_t d = tmem_base + (uint32_t)warp * 128u;
        const long long t0 = clock64();
        for (int i = 0; i < per_issuer; ++i) tc_mma_tf32(d, da + (uint64_t)((i & 3) * 64), db + (uint64_t)((i & 3) * 2), idesc, 1);
        tc_commit(bars + 8 * warp);
        t_issue[warp] = clock64() - t0;
        mbar_wait(bars + 8 * warp, 0, status, 0x401);
        t_done[warp] = clock64() - t0;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        long long a = 0, b = 0;
        for (int w = 0; w < issuers; ++w) {
            a = t_issue[w] > a ? t_issue[w] : a;
            b = t_done[w] > b ? t_done[w] : b;
        }
        out[0] = a;
        out[1] = b;
    }
}

}  // namespace tfb

using namespace tfb;

extern "C" {

tfb_status tfb_probe_mma_issue_cycles(tfb_ctx* ctx, int m, int n, int issuers, double* issue_cycles, double* complete_cycles) {
    if (!ctx || !issue_cycles || !complete_cycles) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_probe_mma_issue_cycles: NULL argument");
    if ((m != 64 && m != 128) || n < 16 || n > 256 || n % 16 != 0 || issuers < 1 || issuers > 4 || (n > 128 && issuers > 1))
        return fail(TFB_ERR_INVALID_ARGUMENT,
                    "tfb_probe_mma_issue_cycles: m is 64 or 128, n a multiple of 16 up to 256 (128 with several issuers), issuers 1..4");
    DeviceGuard g(ctx->device);
    const int per_issuer = 480 / issuers, smem = 64 * 1024 + 1024 + 1024;
    TFB_CUDA(cudaFuncSetAttribute(probe_mma_issue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    PoolBlock out;
    TFB_TRY(out.alloc(ctx, 2 * sizeof(long long)));
    TFB_CUDA(cudaMemsetAsync(out.ptr, 0, 2 * sizeof(long long), ctx->stream));
    {
        LaunchScope ls(ctx, "probe_mma_issue");
        probe_mma_issue_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(issuers, per_issuer, m, n, (long long*)out.ptr, ctx->dev_status);
        TFB_CUDA(cudaGetLastError());
    }
    long long h[2] = {0, 0};
    TFB_CUDA(cudaMemcpyAsync(h, out.ptr, sizeof h, cudaMemcpyDeviceToHost, ctx->stream));
    TFB_CUDA(cudaStreamSynchronize(ctx->stream));
    *issue_cycles = (double)h[0] / per_issuer;      // per MMA, for the thread that issues it
    *complete_cycles = (double)h[1] / (per_issuer * issuers);  // per MMA of the CTA
    return TFB_OK;
}

tfb_status tfb_selftest_wait_expiry(tfb_ctx* ctx, unsigned polls) {
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_selftest_wait_expiry: ctx is NULL");
    if (polls == 0 || polls > (1u << 20))
        return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_selftest_wait_expiry: polls must be in 1..2^20 (a short wait)");
    DeviceGuard g(ctx->device);
    LaunchScope ls(ctx, "selftest_wait_expiry");
    selftest_wait_expiry_kernel<<<1, 32, 0, ctx->stream>>>(ctx->dev_status, polls, nullptr);
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}

tfb_status tfb_probe_fp64_tflops(tfb_ctx* ctx, double* tflops) {
    if (!ctx || !tflops) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_probe_fp64_tflops: NULL argument");
    DeviceGuard g(ctx->device);
    double* sink = nullptr;
    TFB_CUDA(cudaMalloc(&sink, 8));
    const int iters = 20000, grid = ctx->sm_count * 8;
    cudaEvent_t e0, e1;
    TFB_CUDA(cudaEventCreate(&e0));
    TFB_CUDA(cudaEventCreate(&e1));
    double best = 0;
    for (int rep = 0; rep < 4; ++rep) {
        TFB_CUDA(cudaEventRecord(e0, ctx->stream));
        probe_dmma_kernel<<<grid, 256, 0, ctx->stream>>>(sink, iters, 1.0 + rep);
        TFB_CUDA(cudaEventRecord(e1, ctx->stream));
        TFB_CUDA(cudaEventSynchronize(e1));
        float ms = 0;
        TFB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        // warps * DMMAs * 512 flop (8 x 8 x 4 multiply-adds)
        double flop = (double)grid * 8 * (double)iters * 8 * 512.0;
        double t = flop / (ms * 1e-3) / 1e12;
        if (rep > 0 && t > best) best = t;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    *tflops = best;
    return TFB_OK;
}

tfb_status tfb_probe_hbm_gbs(tfb_ctx* ctx, double* gbs) {
    if (!ctx || !gbs) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_probe_hbm_gbs: NULL argument");
    DeviceGuard g(ctx->device);
    const size_t bytes = (size_t)1 << 30;
    uint4 *a = nullptr, *b = nullptr;
    TFB_CUDA(cudaMalloc(&a, bytes));
    if (cudaMalloc(&b, bytes) != cudaSuccess) {
        cudaFree(a);
        return fail(TFB_ERR_DEVICE, "tfb_probe_hbm_gbs: out of memory");
    }
    TFB_CUDA(cudaMemsetAsync(a, 1, bytes, ctx->stream));
    cudaEvent_t e0, e1;
    TFB_CUDA(cudaEventCreate(&e0));
    TFB_CUDA(cudaEventCreate(&e1));
    double best = 0;
    for (int rep = 0; rep < 6; ++rep) {
        TFB_CUDA(cudaEventRecord(e0, ctx->stream));
        probe_copy_kernel<<<ctx->sm_count * 16, 256, 0, ctx->stream>>>(a, b, bytes / 16);
        TFB_CUDA(cudaEventRecord(e1, ctx->stream));
        TFB_CUDA(cudaEventSynchronize(e1));
        float ms = 0;
        TFB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        double t = 2.0 * (double)bytes / (ms * 1e-3) / 1e9;
        if (rep > 0 && t > best) best = t;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(a);
    cudaFree(b);
    *gbs = best;
    return TFB_OK;
}

}  // extern "C"
