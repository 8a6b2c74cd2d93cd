// Grouped f32 products on the tensor cores: the fast path of tfb_grouped_gemm for ragged
// batches of small column-major problems (every dimension a multiple of 16, at most 128
// deep - e.g. 4096 problems with dims drawn from {16, 32, 64, 128}).
//
// Such a batch is bound by HBM (2.7 - 21 flop per byte), not by arithmetic, so the kernel is
// built around moving each operand once: a unit of work is one 64 x 64 output tile of one
// problem with its whole K; persistent CTAs draw unit numbers from an atomic ticket, pull the
// A panel (64 x K) and the B panel (K x 64) into shared memory with 16-byte cp.async, run
// warp-level m16n8k8 TF32 MMAs with the 3xTF32 split done on the fragments in registers, and
// write the tile back through shared memory in full 128-byte lines.  Three CTAs per SM overlap
// one unit's loads with another's arithmetic; nothing ever waits on another CTA.
//
// tcgen05 is the wrong tool here: its 64/128-row tiles would be mostly padding for 16 - 64 row
// problems, and there is no reuse for TMEM to hold.
//
// Semantics: C_p = alpha * A_p B_p + beta * C_p per problem, the formula of
// PrimDescriptor::BatchedGemm (tenferro-prims/src/lib.rs:156-168).
#include <algorithm>

#include "common.h"
#include "contract_common.cuh"

namespace tfb {

namespace {

constexpr int GT = 64;             // output tile
constexpr int GKMAX = 128;         // deepest K the fast path takes
constexpr int LDA = GT + 8;        // [k][m] pitch: fragment reads hit 32 distinct banks
constexpr int kThreads = 128;

struct FastArgs {
    const tfb_gemm_problem* problems;
    const int64_t* unit_prefix;  // [n + 1] units before problem p
    int64_t n_problems, total_units;
    unsigned long long* ticket;
    float alpha, beta;
};

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void split_tf32(float x, uint32_t& big, uint32_t& small) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(big) : "f"(x));
    small = __float_as_uint(x - __uint_as_float(big));
}

__global__ void __launch_bounds__(kThreads, 3) grouped_tf32x3_kernel(FastArgs g) {
    extern __shared__ __align__(16) float smem[];
    float* As = smem;                    // [K][LDA]   (m contiguous, as in memory)
    float* Bs = smem + GKMAX * LDA;      // [64][K + 4] (k contiguous, as in memory)
    __shared__ long long s_unit;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, tq = lane & 3;
    const int wm = (warp & 1) * 32, wn = (warp >> 1) * 32;  // 2 x 2 warps, 32 x 32 each
    for (;;) {
        if (tid == 0) s_unit = (long long)atomicAdd(g.ticket, 1ull);
        __syncthreads();
        const int64_t unit = s_unit;
        if (unit >= g.total_units) break;
        int64_t lo = 0, hi = g.n_problems;
        while (hi - lo > 1) {
            const int64_t mid = (lo + hi) >> 1;
            if (g.unit_prefix[mid] <= unit) lo = mid; else hi = mid;
        }
        const tfb_gemm_problem pr = g.problems[lo];
        const int64_t local = unit - g.unit_prefix[lo];
        const int tiles_m = (int)((pr.m + GT - 1) / GT);
        const int m0 = (int)(local % tiles_m) * GT, n0 = (int)(local / tiles_m) * GT;
        const int M = (int)pr.m, N = (int)pr.n, K = (int)pr.k;
        const int mt = min(GT, M - m0), nt = min(GT, N - n0);  // multiples of 16
        const int LDB = K + 4;
        const float* A = (const float*)pr.a + m0;               // A[m, k] at m + k * a_cs
        const float* B = (const float*)pr.b + (int64_t)n0 * pr.b_cs;  // B[k, n] at k + n * b_cs
        // Panels: 16-byte chunks along the contiguous direction of each operand.
        for (int c = tid; c < K * (mt / 4); c += kThreads) {
            const int k = c / (mt / 4), m4 = (c % (mt / 4)) * 4;
            cp_async_16(As + k * LDA + m4, A + (int64_t)k * pr.a_cs + m4, true);
        }
        for (int c = tid; c < nt * (K / 4); c += kThreads) {
            const int n = c / (K / 4), k4 = (c % (K / 4)) * 4;
            cp_async_16(Bs + n * LDB + k4, B + (int64_t)n * pr.b_cs + k4, true);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        float acc[2][4][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
        const bool warp_live = wm < mt && wn < nt;
        if (warp_live) {
            for (int k0 = 0; k0 < K; k0 += 8) {
                uint32_t ab[2][4], as_[2][4], bb[4][2], bs[4][2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int m = wm + 16 * i + gq;
                    const bool live = m < mt;  // a 16-row half of the warp tile may lie outside the problem
                    const float* p = As + (k0 + tq) * LDA + m;
                    split_tf32(live ? p[0] : 0.f, ab[i][0], as_[i][0]);
                    split_tf32(live ? p[8] : 0.f, ab[i][1], as_[i][1]);
                    split_tf32(live ? p[4 * LDA] : 0.f, ab[i][2], as_[i][2]);
                    split_tf32(live ? p[4 * LDA + 8] : 0.f, ab[i][3], as_[i][3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = wn + 8 * j + gq;
                    const bool live = n < nt;
                    const float* p = Bs + n * LDB + k0 + tq;
                    split_tf32(live ? p[0] : 0.f, bb[j][0], bs[j][0]);
                    split_tf32(live ? p[4] : 0.f, bb[j][1], bs[j][1]);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        mma_tf32(acc[i][j], as_[i], bb[j]);
                        mma_tf32(acc[i][j], ab[i], bs[j]);
                        mma_tf32(acc[i][j], ab[i], bb[j]);
                    }
            }
        }
        __syncthreads();  // panels are dead: reuse the A region as the output tile [n][m]
        float* Cs = smem;
        if (warp_live) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int m = wm + 16 * i + gq, n = wn + 8 * j + 2 * tq;
                    Cs[n * LDA + m] = acc[i][j][0];
                    Cs[(n + 1) * LDA + m] = acc[i][j][1];
                    Cs[n * LDA + m + 8] = acc[i][j][2];
                    Cs[(n + 1) * LDA + m + 8] = acc[i][j][3];
                }
        }
        __syncthreads();
        float* C = (float*)pr.c + m0 + (int64_t)n0 * pr.c_cs;
        const bool read_c = g.beta != 0.f;
        for (int c = tid; c < nt * (mt / 4); c += kThreads) {
            const int n = c / (mt / 4), m4 = (c % (mt / 4)) * 4;
            float4 v = *reinterpret_cast<const float4*>(Cs + n * LDA + m4);
            float4* dst = reinterpret_cast<float4*>(C + (int64_t)n * pr.c_cs + m4);
            v.x *= g.alpha; v.y *= g.alpha; v.z *= g.alpha; v.w *= g.alpha;
            if (read_c) {
                const float4 o = *dst;
                v.x += g.beta * o.x; v.y += g.beta * o.y; v.z += g.beta * o.z; v.w += g.beta * o.w;
            }
            *dst = v;
        }
        __syncthreads();
    }
}

}  // namespace

// Runs the whole table on the tensor-core kernel when every problem qualifies; otherwise
// *declined = true and nothing is launched.
tfb_status grouped_tf32_fast(tfb_ctx* ctx, size_t n, const tfb_gemm_problem* problems, Scalar alpha, Scalar beta,
                             bool* declined) {
    *declined = true;
    if (n == 0 || env_int("TFB_NO_GROUPED_TC", 0)) return TFB_OK;
    if (alpha.im != 0 || beta.im != 0) return TFB_OK;
    std::vector<int64_t> prefix(n + 1, 0);
    for (size_t p = 0; p < n; ++p) {
        const auto& q = problems[p];
        const bool dims_ok = q.m > 0 && q.n > 0 && q.k > 0 && q.m % 16 == 0 && q.n % 16 == 0 && q.k % 16 == 0 && q.k <= GKMAX;
        const bool layout_ok = q.a_rs == 1 && q.b_rs == 1 && q.c_rs == 1 && q.a_cs % 4 == 0 && q.b_cs % 4 == 0 &&
                               q.c_cs % 4 == 0 && q.a_cs >= q.m && q.b_cs >= q.k && q.c_cs >= q.m;
        const bool align_ok = ((uintptr_t)q.a % 16 == 0) && ((uintptr_t)q.b % 16 == 0) && ((uintptr_t)q.c % 16 == 0);
        if (!dims_ok || !layout_ok || !align_ok) return TFB_OK;
        prefix[p + 1] = prefix[p] + ((q.m + GT - 1) / GT) * ((q.n + GT - 1) / GT);
    }
    const int64_t total = prefix[n];
    const size_t bytes_p = n * sizeof(tfb_gemm_problem), bytes_x = (n + 1) * sizeof(int64_t);
    PoolBlock ws;
    TFB_TRY(ws.alloc(ctx, bytes_p + bytes_x + 16));
    char* d = (char*)ws.ptr;
    TFB_CUDA(cudaMemcpyAsync(d, problems, bytes_p, cudaMemcpyHostToDevice, ctx->stream));
    TFB_CUDA(cudaMemcpyAsync(d + bytes_p, prefix.data(), bytes_x, cudaMemcpyHostToDevice, ctx->stream));
    TFB_CUDA(cudaMemsetAsync(d + bytes_p + bytes_x, 0, 16, ctx->stream));
    FastArgs g;
    g.problems = (const tfb_gemm_problem*)d;
    g.unit_prefix = (const int64_t*)(d + bytes_p);
    g.ticket = (unsigned long long*)(d + bytes_p + bytes_x);
    g.n_problems = (int64_t)n;
    g.total_units = total;
    g.alpha = (float)alpha.re;
    g.beta = (float)beta.re;
    const int smem = (GKMAX * LDA + GT * (GKMAX + 4)) * (int)sizeof(float);
    static std::mutex mu;
    static std::map<int, bool> configured;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[ctx->device]) {
            TFB_CUDA(cudaFuncSetAttribute(grouped_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            configured[ctx->device] = true;
        }
    }
    const int grid = (int)std::min<int64_t>(total, (int64_t)ctx->sm_count * 3);
    LaunchScope ls(ctx, "grouped_tf32x3");
    grouped_tf32x3_kernel<<<grid, kThreads, smem, ctx->stream>>>(g);
    TFB_CUDA(cudaGetLastError());
    *declined = false;
    return TFB_OK;
}

}  // namespace tfb
