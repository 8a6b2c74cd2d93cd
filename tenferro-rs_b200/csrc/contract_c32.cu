// Complex32 contraction on the tensor cores as ONE real 3xTF32 product.
//
// A complex product is a real product of doubled extents:
//
//   [ Re C ]   [ Re A  -Im A ] [ Re B ]
//   [ Im C ] = [ Im A   Re A ] [ Im B ]
//
// With the real and imaginary parts interleaved along the rows of C' (row 2m + c), along K of
// both operands (column 2k + c) this reads  C' (2M x N) = A' (2M x 2K) B' (2K x N),  where
//   * C' is the complex output itself, seen as f32: element (m, n) part c lives at float offset
//     2 * offset(m, n) + c, which the kernel's per-row / per-column offset tables express for
//     ANY output strides - so the product is written straight into C, with no planes to recombine;
//   * B' (stored K-major, [n][2k + c]) is the complex operand copied with K fastest - or, when
//     B already has unit stride along a single contracted mode and no conjugation, B itself;
//   * A' is built once by a gather kernel ([2m + c'][2k + c], K-major) with conjugation and the
//     complex alpha folded in.
// Four real products' worth of MMAs instead of the three of the 3M scheme, but no product
// planes (3 x M x N floats written and read again), no cancellation in the imaginary part, and
// one launch of the f32 kernel whatever the output layout.  A complex beta that is not real is
// applied by scaling C first.  A fused multiplier (ContractProblem::mul) is applied to C in
// place after the product.
//
// Semantics: PrimDescriptor::{Contract, BatchedGemm} for Complex32,
// tenferro-prims/src/lib.rs:156-168, 227-239.
#include "contract_common.cuh"
#include "contract_tables.h"

namespace tfb {

namespace {

struct EmbedArgs {
    const float2* src;
    const int64_t* row_tab;  // a_m or b_n
    const int64_t* k_tab;
    const int64_t* b_tab;
    int64_t rows, K, B;
    int64_t ld;              // floats per output row (>= 2K, multiple of 4)
    int src_kfast, conj, embed;
    float2 alpha;
    float* dst;              // embed: [B][2 rows][ld], else [B][rows][ld]
};

// 32 x 32 (rows x k) patches through shared memory: reads follow the source's unit stride,
// writes follow k.  embed = 1 writes the 2 x 2 real block of alpha * op(a) per element (two
// output rows), embed = 0 the element itself.
__global__ void __launch_bounds__(256) embed_operand_kernel(EmbedArgs g) {
    __shared__ float2 tile[32][33];
    const int64_t tiles_r = (g.rows + 31) / 32, tiles_k = (g.K + 31) / 32;
    const int64_t n_tiles = tiles_r * tiles_k * g.B;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const int64_t kpad = g.ld / 2;  // complex columns per output row, zero-filled past K
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
            if (r < g.rows && k < kpad) {
                float2 v = (k < g.K) ? tile[j][tx] : make_float2(0.f, 0.f);
                if (g.conj) v.y = -v.y;
                if (g.embed) {
                    const float2 w = make_float2(g.alpha.x * v.x - g.alpha.y * v.y, g.alpha.x * v.y + g.alpha.y * v.x);
                    float* o = g.dst + ((b * g.rows + r) * 2) * g.ld + 2 * k;
                    *reinterpret_cast<float2*>(o) = make_float2(w.x, -w.y);         // row 2r:     Re, -Im
                    *reinterpret_cast<float2*>(o + g.ld) = make_float2(w.y, w.x);   // row 2r + 1: Im,  Re
                } else {
                    *reinterpret_cast<float2*>(g.dst + (b * g.rows + r) * g.ld + 2 * k) = v;
                }
            }
        }
        __syncthreads();
    }
}

// Offset tables of C seen as f32: row 2m + c -> 2 c_m[m] + c, column n -> 2 c_n[n], batch b -> 2 c_b[b].
__global__ void real_view_tables_kernel(const int64_t* c_m, const int64_t* c_n, const int64_t* c_b, int64_t M, int64_t N,
                                        int64_t B, int64_t* out_m, int64_t* out_n, int64_t* out_b) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 2 * M) out_m[i] = 2 * c_m[i >> 1] + (i & 1);
    if (i < N) out_n[i] = 2 * c_n[i];
    if (i < B) out_b[i] = 2 * c_b[i];
}

// C *= beta (complex), through the tables.
__global__ void __launch_bounds__(256) scale_output_kernel(float2* c, const int64_t* c_b, const int64_t* c_m,
                                                           const int64_t* c_n, int64_t M, int64_t N, int64_t B, float2 beta) {
    const int64_t total = M * N * B, stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t m = idx % M, rest = idx / M, n = rest % N, b = rest / N;
        float2* p = c + c_b[b] + c_m[m] + c_n[n];
        const float2 o = *p;
        *p = make_float2(beta.x * o.x - beta.y * o.y, beta.x * o.y + beta.y * o.x);
    }
}

// B can serve as B' in place when one contracted mode with unit stride carries all of K, nothing
// is conjugated, and every other stride keeps the doubled (float) strides 16-byte aligned.
bool b_is_real_view(const ContractProblem& p) {
    if (p.conj_b || p.k.size() != 1 || p.k[0].s[1] != 1) return false;
    if ((uintptr_t)p.b % 16 != 0 || p.n.size() > 2 || p.batch.size() > 1) return false;
    for (const Mode& m : p.n)
        if (m.extent > 1 && (m.s[1] <= 0 || (2 * m.s[1]) % 4 != 0)) return false;
    for (const Mode& m : p.batch)
        if (m.extent > 1 && (m.s[1] <= 0 || (2 * m.s[1]) % 4 != 0)) return false;
    return true;
}

}  // namespace

static tfb_status embedded_product(tfb_ctx* ctx, const ContractProblem& p, bool* declined) {
    *declined = true;
    if (p.dtype != TFB_C32 || env_int("TFB_NO_TCGEN05", 0)) return TFB_OK;
    const int64_t M = p.M(), N = p.N(), K = p.K(), B = p.B();
    if (2 * M < 32 || N < 32 || K < 4) return TFB_OK;
    const int64_t ld = (2 * K + 3) / 4 * 4;  // rows of the packed operands start on 16-byte boundaries
    if (2 * M * ld * B > (int64_t)1 << 40 || N * ld * B > (int64_t)1 << 40) return TFB_OK;
    std::shared_ptr<ContractTables> t;
    TFB_TRY(get_tables(ctx, p, &t));
    ContractArgs ca;
    fill_args(p, *t, &ca);

    const bool b_in_place = b_is_real_view(p) && env_int("TFB_C32_B_IN_PLACE", 1);
    const size_t a_floats = (size_t)(2 * M * ld * B), b_floats = b_in_place ? 0 : (size_t)(N * ld * B);
    const size_t tab_entries = (size_t)(2 * M + N + B);
    PoolBlock ws;
    TFB_TRY(ws.alloc(ctx, (a_floats + b_floats) * sizeof(float) + tab_entries * sizeof(int64_t) + 256));
    float* a_real = (float*)ws.ptr;
    float* b_real = a_real + a_floats;
    int64_t* tab_m = (int64_t*)(((uintptr_t)(b_real + b_floats) + 15) & ~(uintptr_t)15);
    int64_t* tab_n = tab_m + 2 * M;
    int64_t* tab_b = tab_n + N;

    auto embed = [&](const void* src, const int64_t* row_tab, const int64_t* k_tab, const int64_t* b_tab, int64_t rows,
                     int kfast, bool conj, bool emb, float2 alpha, float* dst) -> tfb_status {
        EmbedArgs g{(const float2*)src, row_tab, k_tab, b_tab, rows, K, B, ld, kfast, conj ? 1 : 0, emb ? 1 : 0, alpha, dst};
        const int64_t n_tiles = ((rows + 31) / 32) * ((K + 31) / 32) * B;
        const int grid = (int)std::min<int64_t>(n_tiles, (int64_t)ctx->sm_count * 16);
        LaunchScope ls(ctx, "pack_planes");
        embed_operand_kernel<<<grid, 256, 0, ctx->stream>>>(g);
        TFB_CUDA(cudaGetLastError());
        return TFB_OK;
    };
    const float2 alpha = make_float2((float)p.alpha.re, (float)p.alpha.im);
    TFB_TRY(embed(p.a, t->a_m, t->a_k, t->a_b, M, ca.a_kfast, p.conj_a, true, alpha, a_real));
    if (!b_in_place)
        TFB_TRY(embed(p.b, t->b_n, t->b_k, t->b_b, N, ca.b_kfast, p.conj_b, false, make_float2(1.f, 0.f), b_real));
    {
        const int64_t n = std::max<int64_t>(std::max<int64_t>(2 * M, N), B);
        real_view_tables_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(t->c_m, t->c_n, t->c_b, M, N, B, tab_m,
                                                                                    tab_n, tab_b);
        count_launch();
        TFB_CUDA(cudaGetLastError());
    }
    double beta = p.beta.re;
    if (p.beta.im != 0) {
        const int64_t blocks = (M * N * B + 255) / 256;
        LaunchScope ls(ctx, "scale");
        scale_output_kernel<<<(unsigned)std::min<int64_t>(blocks, (int64_t)ctx->sm_count * 32), 256, 0, ctx->stream>>>(
            (float2*)p.c, t->c_b, t->c_m, t->c_n, M, N, B, make_float2((float)p.beta.re, (float)p.beta.im));
        TFB_CUDA(cudaGetLastError());
        beta = 1.0;
    }

    // The real product: A' [B][2M][ld] K-major, B' [B][N][ld] K-major (or B itself), C through the tables.
    ContractProblem q;
    q.dtype = TFB_F32;
    q.a = a_real;
    q.b = b_in_place ? p.b : (const void*)b_real;
    q.c = p.c;
    q.alpha = Scalar{1.0, 0.0};
    q.beta = Scalar{beta, 0.0};
    if (b_in_place) {
        if (B > 1) q.batch.push_back(Mode{B, {2 * M * ld, 2 * p.batch[0].s[1], 0}});
        for (const Mode& m : p.n) q.n.push_back(Mode{m.extent, {0, 2 * m.s[1], 0}});
    } else {
        if (B > 1) q.batch.push_back(Mode{B, {2 * M * ld, N * ld, 0}});
        q.n.push_back(Mode{N, {0, ld, 0}});
    }
    q.m.push_back(Mode{2 * M, {ld, 0, 0}});
    q.k.push_back(Mode{2 * K, {1, 1, 0}});
    const int64_t* c_tables[3] = {tab_b, tab_m, tab_n};
    bool d = false;
    TFB_TRY(contract_tcgen05(ctx, q, &d, c_tables, &p.n, 2, &p.m, &p.batch));
    if (d) return fail(TFB_ERR_DEVICE, "internal: the embedded real product was declined by the tensor-core kernel");
    *declined = false;
    return TFB_OK;
}

// Floats the set-up kernels of embedded_product write: the 2 x 2 embedding of the first operand
// (2M x 2K), and a K-major copy of the second (N x 2K) unless it serves in place.
static double setup_floats(const ContractProblem& p) {
    const double k2 = 2.0 * (double)p.K() * (double)p.B();
    return 2.0 * (double)p.M() * k2 + ((b_is_real_view(p) && env_int("TFB_C32_B_IN_PLACE", 1)) ? 0.0 : (double)p.N() * k2);
}

tfb_status contract_c32_embedded(tfb_ctx* ctx, const ContractProblem& p, bool* declined) {
    if (!p.mul) {
        // The embedded operand should be the small one: a tall first operand against a short second
        // one (M >> N) would spend more time being embedded than the product takes.
        if (env_int("TFB_C32_EXCHANGE", 1)) {
            const ContractProblem q = exchange_roles(p);
            if (setup_floats(q) < 0.6 * setup_floats(p)) return embedded_product(ctx, q, declined);
        }
        return embedded_product(ctx, p, declined);
    }
    // A fused multiplier is a complex product per element, and the real embedding holds the two
    // parts of an element in different rows: the product runs unfused and C is multiplied in
    // place afterwards (no intermediate tensor).  With a beta term the exact kernel takes it.
    *declined = true;
    if (!p.beta.is_zero()) return TFB_OK;
    ContractProblem q = p;
    q.mul = nullptr;
    q.conj_mul = false;
    TFB_TRY(embedded_product(ctx, q, declined));
    if (*declined) return TFB_OK;
    std::vector<Mode> all;
    for (auto* g : {&p.m, &p.n, &p.batch})
        for (auto& m : *g) all.push_back(Mode{m.extent, {m.s[2], m.s[3], m.s[2]}});
    sort_and_fuse(all, 2, 3);
    LoopNest nest;
    TFB_TRY(make_nest(all, &nest));
    return launch_elementwise_mul(ctx, p.dtype, nest, p.c, p.mul, p.c, Scalar{1.0, 0.0}, Scalar{0.0, 0.0}, false, p.conj_mul);
}

}  // namespace tfb
