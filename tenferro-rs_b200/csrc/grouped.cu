// Grouped (ragged) matrix products in one persistent launch with a device-side tile
// scheduler.  `PrimDescriptor::BatchedGemm` (tenferro-prims/src/lib.rs:156-168) covers
// uniform batches; a table of problems with individual sizes carries the same
// C = alpha * A * B + beta * C to ragged batches such as 4096 problems with dims drawn
// from {16, 32, 64, 128}.
//
// Scheduling: every problem is cut into 32 x 32 output tiles; tiles are numbered over the
// whole table (a prefix sum per problem) and persistent CTAs draw tile numbers from one
// atomic ticket.  Nothing waits on anything, so the loop needs no bound.
#include <algorithm>

#include "common.h"
#include "scalar_ops.cuh"

namespace tfb {

struct GroupedArgs {
    const tfb_gemm_problem* problems;  // device copy
    const int64_t* tile_prefix;        // [n + 1] tiles before problem p
    int64_t n_problems, total_tiles;
    unsigned long long* ticket;
    double alpha_re, alpha_im, beta_re, beta_im;
};

constexpr int GT = 32, GK = 16;

template <typename T>
__global__ void __launch_bounds__(64) grouped_simt_kernel(GroupedArgs g) {
    __shared__ T As[GK][GT + 1];
    __shared__ T Bs[GK][GT + 1];
    __shared__ long long s_tile;
    const int tid = threadIdx.x;
    const int tx = tid & 7, ty = tid >> 3;  // 8 x 8 threads, 4 x 4 outputs each
    const T alpha = Ops<T>::from(Scalar{g.alpha_re, g.alpha_im});
    const T beta = Ops<T>::from(Scalar{g.beta_re, g.beta_im});
    const bool read_c = g.beta_re != 0 || g.beta_im != 0;
    for (;;) {
        if (tid == 0) s_tile = (long long)atomicAdd(g.ticket, 1ull);
        __syncthreads();
        const int64_t tile = s_tile;
        __syncthreads();
        if (tile >= g.total_tiles) break;
        // Problem of this tile: last p with tile_prefix[p] <= tile.
        int64_t lo = 0, hi = g.n_problems;
        while (hi - lo > 1) {
            int64_t mid = (lo + hi) >> 1;
            if (g.tile_prefix[mid] <= tile) lo = mid; else hi = mid;
        }
        const tfb_gemm_problem pr = g.problems[lo];
        const int64_t local = tile - g.tile_prefix[lo];
        const int64_t tiles_m = (pr.m + GT - 1) / GT;
        const int64_t m0 = (local % tiles_m) * GT, n0 = (local / tiles_m) * GT;
        const T* A = (const T*)pr.a;
        const T* B = (const T*)pr.b;
        T* C = (T*)pr.c;
        // Threads follow whichever direction of each operand has the smaller stride.
        const bool a_kfast = llabs(pr.a_cs) < llabs(pr.a_rs), b_kfast = llabs(pr.b_rs) < llabs(pr.b_cs);
        T acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = Ops<T>::zero();
        for (int64_t k0 = 0; k0 < pr.k; k0 += GK) {
#pragma unroll
            for (int r = 0; r < GT * GK / 64; ++r) {
                int c = tid + r * 64;
                int mm, kk;
                if (a_kfast) { kk = c % GK; mm = c / GK; } else { mm = c % GT; kk = c / GT; }
                T v = Ops<T>::zero();
                if (m0 + mm < pr.m && k0 + kk < pr.k) v = A[(m0 + mm) * pr.a_rs + (k0 + kk) * pr.a_cs];
                As[kk][mm] = v;
                int nn;
                if (b_kfast) { kk = c % GK; nn = c / GK; } else { nn = c % GT; kk = c / GT; }
                T w = Ops<T>::zero();
                if (n0 + nn < pr.n && k0 + kk < pr.k) w = B[(k0 + kk) * pr.b_rs + (n0 + nn) * pr.b_cs];
                Bs[kk][nn] = w;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < GK; ++kk) {
                T av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) av[i] = As[kk][tx + 8 * i];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][ty + 8 * j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = Ops<T>::fma_(av[i], bv[j], acc[i][j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t n = n0 + ty + 8 * j;
            if (n >= pr.n) continue;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t m = m0 + tx + 8 * i;
                if (m >= pr.m) continue;
                T* p = C + m * pr.c_rs + n * pr.c_cs;
                T v = Ops<T>::mul(alpha, acc[i][j]);
                if (read_c) v = Ops<T>::add(v, Ops<T>::mul(beta, *p));
                *p = v;
            }
        }
    }
}

tfb_status grouped_simt(tfb_ctx* ctx, int dtype, size_t n, const tfb_gemm_problem* problems, Scalar alpha, Scalar beta) {
    if (n == 0) return TFB_OK;
    std::vector<int64_t> prefix(n + 1, 0);
    for (size_t p = 0; p < n; ++p) {
        const auto& q = problems[p];
        if (q.m < 0 || q.n < 0 || q.k < 0) return fail(TFB_ERR_INVALID_ARGUMENT, "problem %zu has a negative size", p);
        if (q.m > 0 && q.n > 0 && (!q.c || (q.k > 0 && (!q.a || !q.b))))
            return fail(TFB_ERR_INVALID_ARGUMENT, "problem %zu has a NULL pointer", p);
        prefix[p + 1] = prefix[p] + ((q.m + GT - 1) / GT) * ((q.n + GT - 1) / GT);
    }
    const int64_t total = prefix[n];
    if (total == 0) return TFB_OK;
    // One scratch block: problems | prefix | ticket.
    const size_t bytes_p = n * sizeof(tfb_gemm_problem), bytes_x = (n + 1) * sizeof(int64_t);
    PoolBlock ws;
    TFB_TRY(ws.alloc(ctx, bytes_p + bytes_x + 16));
    char* d = (char*)ws.ptr;
    TFB_CUDA(cudaMemcpyAsync(d, problems, bytes_p, cudaMemcpyHostToDevice, ctx->stream));
    TFB_CUDA(cudaMemcpyAsync(d + bytes_p, prefix.data(), bytes_x, cudaMemcpyHostToDevice, ctx->stream));
    TFB_CUDA(cudaMemsetAsync(d + bytes_p + bytes_x, 0, 16, ctx->stream));
    // The host vectors above are pageable: the copies have been staged by the time the calls return.
    GroupedArgs g;
    g.problems = (const tfb_gemm_problem*)d;
    g.tile_prefix = (const int64_t*)(d + bytes_p);
    g.ticket = (unsigned long long*)(d + bytes_p + bytes_x);
    g.n_problems = (int64_t)n;
    g.total_tiles = total;
    g.alpha_re = alpha.re; g.alpha_im = alpha.im; g.beta_re = beta.re; g.beta_im = beta.im;
    const int grid = (int)std::min<int64_t>(total, (int64_t)ctx->sm_count * 16);
    LaunchScope ls(ctx, "grouped_simt");
    switch (dtype) {
        case TFB_F32: grouped_simt_kernel<float><<<grid, 64, 0, ctx->stream>>>(g); break;
        case TFB_F64: grouped_simt_kernel<double><<<grid, 64, 0, ctx->stream>>>(g); break;
        case TFB_C32: grouped_simt_kernel<float2><<<grid, 64, 0, ctx->stream>>>(g); break;
        case TFB_C64: grouped_simt_kernel<double2><<<grid, 64, 0, ctx->stream>>>(g); break;
        default: return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    }
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}

}  // namespace tfb

// A problem table prepared once: the tensor-core schedule on the device when the table
// qualifies, else the host copy of the table for the SIMT kernel.
struct tfb_grouped_plan {
    tfb_ctx* ctx = nullptr;
    int dtype = 0;
    bool fast = false;
    tfb::GroupedFast schedule;
    std::vector<tfb_gemm_problem> problems;
};

namespace {

tfb_status prepare(tfb_ctx* ctx, int dtype, size_t n, const tfb_gemm_problem* problems, tfb_grouped_plan* plan) {
    using namespace tfb;
    DeviceGuard g(ctx->device);
    plan->ctx = ctx;
    plan->dtype = dtype;
    plan->problems.assign(problems, problems + n);
    if (dtype == TFB_F32) {
        // The mma.sync kernel is the faster one on the tables it takes (dims in multiples of 16, K up to
        // 128); the tcgen05 kernel takes any dims with 16-byte aligned columns and K up to 512; the
        // SIMT kernel takes everything.
        const bool tcgen05_first = env_int("TFB_GROUPED_PREFER_TCGEN05", 0) != 0;
        bool declined = true;
        if (tcgen05_first) TFB_TRY(grouped_tcgen05_prepare(ctx, n, problems, &plan->schedule, &declined));
        if (declined) TFB_TRY(grouped_tf32_prepare(ctx, n, problems, &plan->schedule, &declined));
        if (declined && !tcgen05_first) TFB_TRY(grouped_tcgen05_prepare(ctx, n, problems, &plan->schedule, &declined));
        plan->fast = !declined;
    }
    return TFB_OK;
}

tfb_status run(tfb_grouped_plan* plan, tfb::Scalar alpha, tfb::Scalar beta) {
    using namespace tfb;
    DeviceGuard g(plan->ctx->device);
    if (plan->fast) {
        bool declined = true;
        if (plan->schedule.tcgen05)
            TFB_TRY(grouped_tcgen05_run(plan->ctx, plan->schedule, alpha, beta, &declined));
        else
            TFB_TRY(grouped_tf32_run(plan->ctx, plan->schedule, alpha, beta, &declined));
        if (!declined) return TFB_OK;
    }
    return grouped_simt(plan->ctx, plan->dtype, plan->problems.size(), plan->problems.data(), alpha, beta);
}

tfb_status check_args(const char* who, tfb_ctx* ctx, int32_t dtype, size_t n, const tfb_gemm_problem* problems) {
    using namespace tfb;
    if (!ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: ctx is NULL", who);
    if (!dtype_valid(dtype)) return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", (int)dtype);
    if (n && !problems) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: problems is NULL", who);
    return TFB_OK;
}

}  // namespace

extern "C" tfb_status tfb_grouped_gemm(tfb_ctx* ctx, int32_t dtype, size_t n_problems, const tfb_gemm_problem* problems,
                                       const void* alpha, const void* beta) {
    using namespace tfb;
    TFB_TRY(check_args("tfb_grouped_gemm", ctx, dtype, n_problems, problems));
    if (!alpha || !beta) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_grouped_gemm: alpha/beta are NULL");
    tfb_grouped_plan plan;
    TFB_TRY(prepare(ctx, dtype, n_problems, problems, &plan));
    return run(&plan, load_scalar(dtype, alpha), load_scalar(dtype, beta));
}

extern "C" tfb_status tfb_grouped_plan_create(tfb_ctx* ctx, int32_t dtype, size_t n_problems,
                                              const tfb_gemm_problem* problems, tfb_grouped_plan** out) {
    using namespace tfb;
    TFB_TRY(check_args("tfb_grouped_plan_create", ctx, dtype, n_problems, problems));
    if (!out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_grouped_plan_create: out is NULL");
    auto* plan = new (std::nothrow) tfb_grouped_plan;
    if (!plan) return fail(TFB_ERR_DEVICE, "out of host memory");
    const tfb_status st = prepare(ctx, dtype, n_problems, problems, plan);
    if (st != TFB_OK) {
        delete plan;
        return st;
    }
    *out = plan;
    return TFB_OK;
}

extern "C" tfb_status tfb_grouped_plan_execute(tfb_grouped_plan* plan, const void* alpha, const void* beta) {
    using namespace tfb;
    if (!plan) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_grouped_plan_execute: plan is NULL");
    if (!alpha || !beta) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_grouped_plan_execute: alpha/beta are NULL");
    return run(plan, load_scalar(plan->dtype, alpha), load_scalar(plan->dtype, beta));
}

extern "C" void tfb_grouped_plan_destroy(tfb_grouped_plan* plan) { delete plan; }
