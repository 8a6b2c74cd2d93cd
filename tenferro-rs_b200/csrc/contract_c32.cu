// Complex32 contraction on the tensor cores: three real 3xTF32 products (the "3M" scheme)
// around the f32 tcgen05 kernel.
//
//   P1 = Ar Br,  P2 = Ai Bi,  P3 = (Ar + Ai)(Br + Bi)
//   Re C = P1 - P2,   Im C = P3 - P1 - P2
//
// A gather kernel reads the interleaved operands through the offset tables (any strides, conj
// folded in as a sign) and writes the three real planes of each operand K-major, the layout
// the tensor-core kernel streams fastest; a scatter kernel combines the three products,
// applies alpha/beta in complex arithmetic and writes the interleaved output through the C
// tables.  The planes and products live in pool scratch for the duration of the call.
// One fewer product than the textbook four; the subtraction in Im C costs about a factor
// of three in rounding error, which 3xTF32 (1e-6) has to spare against the 1e-5 tolerance.
//
// Semantics: PrimDescriptor::{Contract, BatchedGemm} for Complex32,
// tenferro-prims/src/lib.rs:156-168, 227-239.
#include "contract_common.cuh"
#include "contract_tables.h"

namespace tfb {

namespace {

struct PackArgs {
    const float2* src;
    const int64_t* row_tab;  // a_m or b_n
    const int64_t* k_tab;
    const int64_t* b_tab;
    int64_t rows, K, Kp, B;
    int src_kfast, conj;
    float* re;
    float* im;
    float* sum;
};

// 32 x 32 (rows x k) patches through shared memory: reads follow the source's unit stride,
// writes follow k.
__global__ void __launch_bounds__(256) pack_planes_kernel(PackArgs g) {
    __shared__ float2 tile[32][33];
    const int64_t tiles_r = (g.rows + 31) / 32, tiles_k = (g.K + 31) / 32;
    const int64_t n_tiles = tiles_r * tiles_k * g.B;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int64_t tr = t % tiles_r, rest = t / tiles_r, tk = rest % tiles_k, b = rest / tiles_k;
        const int64_t r0 = tr * 32, k0 = tk * 32;
        const float2* src = g.src + g.b_tab[b];
        for (int j = ty; j < 32; j += 8) {
            // (r, k) of this thread's element: tx runs along the source's fast direction
            const int64_t r = r0 + (g.src_kfast ? j : tx), k = k0 + (g.src_kfast ? tx : j);
            float2 v = make_float2(0.f, 0.f);
            if (r < g.rows && k < g.K) v = src[g.row_tab[r] + g.k_tab[k]];
            if (g.src_kfast) tile[j][tx] = v; else tile[tx][j] = v;  // tile[r][k]
        }
        __syncthreads();
        for (int j = ty; j < 32; j += 8) {
            const int64_t r = r0 + j, k = k0 + tx;
            if (r < g.rows && k < g.Kp) {
                float2 v = (k < g.K) ? tile[j][tx] : make_float2(0.f, 0.f);
                if (g.conj) v.y = -v.y;
                const int64_t o = (b * g.rows + r) * g.Kp + k;
                g.re[o] = v.x;
                g.im[o] = v.y;
                g.sum[o] = v.x + v.y;
            }
        }
        __syncthreads();
    }
}

struct UnpackArgs {
    const float* p1;
    const float* p2;
    const float* p3;
    float2* c;
    const int64_t* c_b;
    const int64_t* c_m;
    const int64_t* c_n;
    int64_t M, N, B;
    float2 alpha, beta;
};

__global__ void __launch_bounds__(256) unpack_products_kernel(UnpackArgs g) {
    const int64_t total = g.M * g.N * g.B;
    const bool read_c = g.beta.x != 0.f || g.beta.y != 0.f;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t m = idx % g.M, rest = idx / g.M, n = rest % g.N, b = rest / g.N;
        const float a = g.p1[idx], bb = g.p2[idx], s = g.p3[idx];
        const float re = a - bb, im = s - a - bb;
        float2* p = g.c + g.c_b[b] + g.c_m[m] + g.c_n[n];
        float2 o = make_float2(g.alpha.x * re - g.alpha.y * im, g.alpha.x * im + g.alpha.y * re);
        if (read_c) {
            const float2 old = *p;
            o.x += g.beta.x * old.x - g.beta.y * old.y;
            o.y += g.beta.x * old.y + g.beta.y * old.x;
        }
        *p = o;
    }
}

}  // namespace

tfb_status contract_c32_3m(tfb_ctx* ctx, const ContractProblem& p, bool* declined) {
    *declined = true;
    if (p.dtype != TFB_C32 || env_int("TFB_NO_TCGEN05", 0)) return TFB_OK;
    const int64_t M = p.M(), N = p.N(), K = p.K(), B = p.B();
    if (M < 32 || N < 32 || K < 8) return TFB_OK;
    const int64_t Kp = (K + 3) / 4 * 4;  // rows of the planes start on 16-byte boundaries
    if (M * Kp * B > (int64_t)1 << 40 || N * Kp * B > (int64_t)1 << 40) return TFB_OK;
    std::shared_ptr<ContractTables> t;
    TFB_TRY(get_tables(ctx, p, &t));
    ContractArgs ca;
    fill_args(p, *t, &ca);

    const size_t a_plane = (size_t)(M * Kp * B), b_plane = (size_t)(N * Kp * B), c_plane = (size_t)(M * N * B);
    PoolBlock ws;
    TFB_TRY(ws.alloc(ctx, (3 * a_plane + 3 * b_plane + 3 * c_plane) * sizeof(float) + 256));
    float* base = (float*)ws.ptr;
    float *ar = base, *ai = ar + a_plane, *as = ai + a_plane;
    float *br = as + a_plane, *bi = br + b_plane, *bs = bi + b_plane;
    float *p1 = bs + b_plane, *p2 = p1 + c_plane, *p3 = p2 + c_plane;

    auto pack = [&](const void* src, const int64_t* row_tab, const int64_t* k_tab, const int64_t* b_tab, int64_t rows,
                    int kfast, bool conj, float* re, float* im, float* sum) -> tfb_status {
        PackArgs g{(const float2*)src, row_tab, k_tab, b_tab, rows, K, Kp, B, kfast, conj ? 1 : 0, re, im, sum};
        const int64_t n_tiles = ((rows + 31) / 32) * ((K + 31) / 32) * B;
        const int grid = (int)std::min<int64_t>(n_tiles, (int64_t)ctx->sm_count * 16);
        LaunchScope ls(ctx, "pack_planes");
        pack_planes_kernel<<<grid, 256, 0, ctx->stream>>>(g);
        TFB_CUDA(cudaGetLastError());
        return TFB_OK;
    };
    TFB_TRY(pack(p.a, t->a_m, t->a_k, t->a_b, M, ca.a_kfast, p.conj_a, ar, ai, as));
    TFB_TRY(pack(p.b, t->b_n, t->b_k, t->b_b, N, ca.b_kfast, p.conj_b, br, bi, bs));

    // Three real products on the packed planes: A' [B][M][Kp] and B' [B][N][Kp] K-major, P [B][N][M].
    auto product = [&](const float* a, const float* b, float* c) -> tfb_status {
        ContractProblem q;
        q.dtype = TFB_F32;
        q.a = a; q.b = b; q.c = c;
        q.alpha = Scalar{1.0, 0.0};
        q.beta = Scalar{0.0, 0.0};
        if (B > 1) q.batch.push_back(Mode{B, {M * Kp, N * Kp, M * N}});
        q.m.push_back(Mode{M, {Kp, 0, 1}});
        q.n.push_back(Mode{N, {0, Kp, M}});
        q.k.push_back(Mode{K, {1, 1, 0}});
        bool d = false;
        TFB_TRY(contract_tcgen05(ctx, q, &d));
        if (d) return fail(TFB_ERR_DEVICE, "internal: the packed real product was declined by the tensor-core kernel");
        return TFB_OK;
    };
    TFB_TRY(product(ar, br, p1));
    TFB_TRY(product(ai, bi, p2));
    TFB_TRY(product(as, bs, p3));

    UnpackArgs u{p1, p2, p3, (float2*)p.c, t->c_b, t->c_m, t->c_n, M, N, B,
                 make_float2((float)p.alpha.re, (float)p.alpha.im), make_float2((float)p.beta.re, (float)p.beta.im)};
    const int64_t blocks = (M * N * B + 255) / 256;
    const int grid = (int)std::min<int64_t>(blocks, (int64_t)ctx->sm_count * 32);
    {
        LaunchScope ls(ctx, "unpack_products");
        unpack_products_kernel<<<grid, 256, 0, ctx->stream>>>(u);
    }
    TFB_CUDA(cudaGetLastError());
    *declined = false;
    return TFB_OK;
}

}  // namespace tfb
