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

}  // namespace tfb

using namespace tfb;

extern "C" {

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
