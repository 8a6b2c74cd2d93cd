// Contraction driver: offset tables, kernel selection, and the SIMT kernel that takes
// whatever the tensor-core kernels decline.  Implements the arithmetic of
// `PrimDescriptor::{Contract, BatchedGemm}` (tenferro-prims/src/lib.rs:156-168, 227-239).
#include "contract_common.cuh"
#include "contract_tables.h"
#include "scalar_ops.cuh"

namespace tfb {

static int64_t prod(const std::vector<Mode>& v) {
    int64_t p = 1;
    for (auto& m : v) p *= m.extent;
    return p;
}
int64_t ContractProblem::M() const { return prod(m); }
int64_t ContractProblem::N() const { return prod(n); }
int64_t ContractProblem::K() const { return prod(k); }
int64_t ContractProblem::B() const { return prod(batch); }

// ------------------------------------------------------------------ offset tables
struct TableJob {
    LoopNest nest;     // the group's modes, strides for tensors 0..2
    int64_t* out[3];   // table per tensor (nullptr: tensor does not carry this group)
};
struct TableJobs {
    TableJob job[4];
};

__global__ void __launch_bounds__(256) build_tables_kernel(TableJobs jobs) {
    const TableJob& j = jobs.job[blockIdx.y];
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < j.nest.total; idx += stride) {
        int64_t rem = idx, off0 = 0, off1 = 0, off2 = 0;
        for (int d = 0; d < j.nest.rank; ++d) {
            int64_t q = rem / j.nest.extent[d];
            int64_t r = rem - q * j.nest.extent[d];
            off0 += r * j.nest.stride[0][d];
            off1 += r * j.nest.stride[1][d];
            off2 += r * j.nest.stride[2][d];
            rem = q;
        }
        if (j.out[0]) j.out[0][idx] = off0;
        if (j.out[1]) j.out[1][idx] = off1;
        if (j.out[2]) j.out[2][idx] = off2;
    }
}

ContractTables::~ContractTables() {
    if (block) cudaFree(block);
    if (built) cudaEventDestroy(built);
}

static std::string signature(const ContractProblem& p) {
    std::string s;
    auto put = [&](const std::vector<Mode>& g) {
        int64_t n = (int64_t)g.size();
        s.append((const char*)&n, sizeof n);
        for (auto& m : g) s.append((const char*)&m, sizeof m);
    };
    put(p.batch);
    put(p.m);
    put(p.n);
    put(p.k);
    s.push_back(p.mul ? 'd' : '-');
    return s;
}

struct TableCache {
    std::mutex mu;
    std::map<std::pair<int, std::string>, std::shared_ptr<ContractTables>> map;
    std::vector<std::pair<int, std::string>> order;
};
static TableCache& cache() {
    static TableCache c;
    return c;
}

tfb_status get_tables(tfb_ctx* ctx, const ContractProblem& p, std::shared_ptr<ContractTables>* out) {
    auto key = std::make_pair(ctx->device, signature(p));
    TableCache& tc = cache();
    std::lock_guard<std::mutex> lock(tc.mu);
    auto it = tc.map.find(key);
    if (it != tc.map.end()) {
        ContractTables& hit = *it->second;
        // Same stream as the build: stream order is enough.  Any other stream (another context
        // of this device, or this context after tfb_ctx_set_stream) must not read the tables
        // before the kernels that fill them have run.
        if (!hit.ready && hit.built) {
            if (cudaEventQuery(hit.built) == cudaSuccess) {
                hit.ready = true;
            } else {
                cudaGetLastError();
                if (ctx->stream != hit.build_stream) TFB_CUDA(cudaStreamWaitEvent(ctx->stream, hit.built, 0));
            }
        }
        *out = it->second;
        return TFB_OK;
    }
    auto t = std::make_shared<ContractTables>();
    t->M = p.M();
    t->N = p.N();
    t->K = p.K();
    t->B = p.B();
    // One allocation: a_b b_b c_b | a_m c_m | b_n c_n | a_k b_k | d_b d_m d_n
    size_t n_entries = (size_t)(3 * t->B + 2 * t->M + 2 * t->N + 2 * t->K);
    if (p.mul) n_entries += (size_t)(t->B + t->M + t->N);
    TFB_CUDA(cudaMalloc(&t->block, n_entries * sizeof(int64_t) + 64));
    int64_t* q = (int64_t*)t->block;
    t->a_b = q; q += t->B;
    t->b_b = q; q += t->B;
    t->c_b = q; q += t->B;
    t->a_m = q; q += t->M;
    t->c_m = q; q += t->M;
    t->b_n = q; q += t->N;
    t->c_n = q; q += t->N;
    t->a_k = q; q += t->K;
    t->b_k = q; q += t->K;
    if (p.mul) {
        t->d_b = q; q += t->B;
        t->d_m = q; q += t->M;
        t->d_n = q; q += t->N;
    }
    TableJobs jobs;
    TFB_TRY(make_nest(p.batch, &jobs.job[0].nest));
    jobs.job[0].out[0] = t->a_b; jobs.job[0].out[1] = t->b_b; jobs.job[0].out[2] = t->c_b;
    TFB_TRY(make_nest(p.m, &jobs.job[1].nest));
    jobs.job[1].out[0] = t->a_m; jobs.job[1].out[1] = nullptr; jobs.job[1].out[2] = t->c_m;
    TFB_TRY(make_nest(p.n, &jobs.job[2].nest));
    jobs.job[2].out[0] = nullptr; jobs.job[2].out[1] = t->b_n; jobs.job[2].out[2] = t->c_n;
    TFB_TRY(make_nest(p.k, &jobs.job[3].nest));
    jobs.job[3].out[0] = t->a_k; jobs.job[3].out[1] = t->b_k; jobs.job[3].out[2] = nullptr;
    int64_t biggest = std::max(std::max(t->B, t->M), std::max(t->N, t->K));
    int gx = (int)std::min<int64_t>((biggest + 255) / 256, 1024);
    if (gx < 1) gx = 1;
    LaunchScope ls(ctx, "build_tables");
    build_tables_kernel<<<dim3(gx, 4), 256, 0, ctx->stream>>>(jobs);
    TFB_CUDA(cudaGetLastError());
    if (p.mul) {
        // The multiplier's offsets over the same three output groups (its strides are slot 3).
        auto slot3 = [](const std::vector<Mode>& g) {
            std::vector<Mode> r;
            for (auto& m : g) r.push_back(Mode{m.extent, {m.s[3], 0, 0}});
            return r;
        };
        TableJobs dj;
        TFB_TRY(make_nest(slot3(p.batch), &dj.job[0].nest));
        TFB_TRY(make_nest(slot3(p.m), &dj.job[1].nest));
        TFB_TRY(make_nest(slot3(p.n), &dj.job[2].nest));
        TFB_TRY(make_nest(std::vector<Mode>{}, &dj.job[3].nest));
        dj.job[3].nest.total = 0;
        for (int j = 0; j < 4; ++j) dj.job[j].out[0] = dj.job[j].out[1] = dj.job[j].out[2] = nullptr;
        dj.job[0].out[0] = t->d_b;
        dj.job[1].out[0] = t->d_m;
        dj.job[2].out[0] = t->d_n;
        build_tables_kernel<<<dim3(gx, 4), 256, 0, ctx->stream>>>(dj);
        count_launch();
        TFB_CUDA(cudaGetLastError());
    }
    TFB_CUDA(cudaEventCreateWithFlags(&t->built, cudaEventDisableTiming));
    TFB_CUDA(cudaEventRecord(t->built, ctx->stream));
    t->build_stream = ctx->stream;
    // Bounded cache: drop the oldest entry once 256 layouts are held.  Tables in use by
    // enqueued kernels stay alive through cudaFree's implicit synchronisation.
    if (tc.order.size() >= 256) {
        tc.map.erase(tc.order.front());
        tc.order.erase(tc.order.begin());
    }
    tc.map[key] = t;
    tc.order.push_back(key);
    *out = t;
    return TFB_OK;
}

// Unit-stride analysis of one operand tile: is the group's first (fastest) mode stride 1 in
// tensor `t`, and can two f64 travel as one 16-byte chunk?
static bool group_unit_stride(const std::vector<Mode>& g, int t) { return !g.empty() && g[0].s[t] == 1; }
static bool all_even(const std::vector<Mode>& g, int t, size_t from) {
    for (size_t i = from; i < g.size(); ++i)
        if (g[i].s[t] % 2 != 0) return false;
    return true;
}

void fill_args(const ContractProblem& p, const ContractTables& t, ContractArgs* a) {
    memset(a, 0, sizeof *a);
    a->a = (const char*)p.a;
    a->b = (const char*)p.b;
    a->c = (char*)p.c;
    a->a_b = t.a_b; a->b_b = t.b_b; a->c_b = t.c_b;
    a->a_m = t.a_m; a->c_m = t.c_m;
    a->b_n = t.b_n; a->c_n = t.c_n;
    a->a_k = t.a_k; a->b_k = t.b_k;
    a->M = t.M; a->N = t.N; a->K = t.K; a->B = t.B;
    a->alpha_re = p.alpha.re; a->alpha_im = p.alpha.im;
    a->beta_re = p.beta.re; a->beta_im = p.beta.im;
    a->conj_a = p.conj_a && dtype_is_complex(p.dtype);
    a->conj_b = p.conj_b && dtype_is_complex(p.dtype);
    a->mul = (const char*)p.mul;
    a->d_b = t.d_b; a->d_m = t.d_m; a->d_n = t.d_n;
    a->conj_mul = p.conj_mul && dtype_is_complex(p.dtype);
    // Direction of the unit stride in each operand tile.  If neither group is unit-stride
    // the choice only affects which threads sit next to each other.
    bool a_k1 = group_unit_stride(p.k, 0), a_m1 = group_unit_stride(p.m, 0);
    bool b_k1 = group_unit_stride(p.k, 1), b_n1 = group_unit_stride(p.n, 1);
    a->a_kfast = a_k1 || !a_m1;
    a->b_kfast = b_k1 || !b_n1;
    a->a_vec = a->b_vec = 1;
    if (p.dtype == TFB_F64) {
        // 16-byte chunks of two doubles along the unit-stride group: its first extent must be
        // even, every other stride of that operand even, and the element pointer 16-byte aligned.
        auto pair_ok = [&](const std::vector<Mode>& fast, const std::vector<Mode>& other, int tns, const void* base) {
            if (fast.empty() || fast[0].s[tns] != 1 || fast[0].extent % 2 != 0) return false;
            if (!all_even(fast, tns, 1) || !all_even(other, tns, 0) || !all_even(p.batch, tns, 0)) return false;
            return (uintptr_t)base % 16 == 0;
        };
        if (a->a_kfast ? pair_ok(p.k, p.m, 0, p.a) : pair_ok(p.m, p.k, 0, p.a)) a->a_vec = 2;
        if (a->b_kfast ? pair_ok(p.k, p.n, 1, p.b) : pair_ok(p.n, p.k, 1, p.b)) a->b_vec = 2;
    }
}

// ------------------------------------------------------------------ SIMT kernel
// 64 x 64 block tile, 16-deep k slices, 256 threads, 4 x 4 outputs per thread.  Exact in
// the element type (FMA), any strides, any dtype.  It is the path of last resort: the
// tensor-core kernels decline only layouts they cannot stage.
// ALG selects the semiring (scalar_ops.cuh): the same loop nest computes
// C = alpha (x) (+)_k A (x) B  (+)  beta (x) C for MaxPlus and MinPlus, which have no tensor-core form.
template <typename T, int ALG = 0>
__global__ void __launch_bounds__(256) contract_simt_kernel(ContractArgs g) {
    using S = Semi<T, ALG>;
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ T As[BK][BM + 1];
    __shared__ T Bs[BK][BN + 1];
    const T* A = (const T*)g.a;
    const T* Bp = (const T*)g.b;
    T* C = (T*)g.c;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 x 4
    for (int64_t tile = blockIdx.x; tile < g.n_tiles; tile += gridDim.x) {
        int64_t tm = tile % g.tiles_m;
        int64_t rest = tile / g.tiles_m;
        int64_t tn = rest % g.tiles_n;
        int64_t bb = rest / g.tiles_n;
        const int64_t m0 = tm * BM, n0 = tn * BN;
        const T* Ab = A + g.a_b[bb];
        const T* Bb = Bp + g.b_b[bb];
        T acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = S::zero();
        for (int64_t k0 = 0; k0 < g.K; k0 += BK) {
            // Gather the two operand slices; neighbouring threads follow the unit stride.
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                int c = tid + r * 256;
                int mm, kk;
                if (g.a_kfast) { kk = c % BK; mm = c / BK; } else { mm = c % BM; kk = c / BM; }
                T v = S::zero();
                if (m0 + mm < g.M && k0 + kk < g.K) v = Ab[g.a_m[m0 + mm] + g.a_k[k0 + kk]];
                if (g.conj_a) v = Ops<T>::conj(v);
                As[kk][mm] = v;
                int nn;
                if (g.b_kfast) { kk = c % BK; nn = c / BK; } else { nn = c % BN; kk = c / BN; }
                T w = S::zero();
                if (n0 + nn < g.N && k0 + kk < g.K) w = Bb[g.b_n[n0 + nn] + g.b_k[k0 + kk]];
                if (g.conj_b) w = Ops<T>::conj(w);
                Bs[kk][nn] = w;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                T av[4], bv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) av[i] = As[kk][tx + 16 * i];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][ty + 16 * j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = S::fma_(av[i], bv[j], acc[i][j]);
            }
            __syncthreads();
        }
        const T alpha = Ops<T>::from(Scalar{g.alpha_re, g.alpha_im});
        const T beta = Ops<T>::from(Scalar{g.beta_re, g.beta_im});
        // beta equal to the semiring's zero means "overwrite": the output is never read
        const bool read_c = ALG == 0 ? (g.beta_re != 0 || g.beta_im != 0) : !(g.beta_re == (ALG == 1 ? -INFINITY : INFINITY));
        T* Cb = C + g.c_b[bb];
        const T* D = g.mul ? reinterpret_cast<const T*>(g.mul) + g.d_b[bb] : nullptr;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int64_t n = n0 + ty + 16 * j;
            if (n >= g.N) continue;
            int64_t cn = g.c_n[n];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int64_t m = m0 + tx + 16 * i;
                if (m >= g.M) continue;
                T* p = Cb + g.c_m[m] + cn;
                T sum = acc[i][j];
                if (D) {
                    const T d = D[g.d_m[m] + g.d_n[n]];
                    sum = Ops<T>::mul(sum, g.conj_mul ? Ops<T>::conj(d) : d);
                }
                T v = S::mul(alpha, sum);
                if (read_c) v = S::add(v, S::mul(beta, *p));
                *p = v;
            }
        }
    }
}

tfb_status contract_simt(tfb_ctx* ctx, const ContractProblem& p) {
    std::shared_ptr<ContractTables> t;
    TFB_TRY(get_tables(ctx, p, &t));
    ContractArgs a;
    fill_args(p, *t, &a);
    a.tiles_m = (a.M + 63) / 64;
    a.tiles_n = (a.N + 63) / 64;
    a.n_tiles = a.tiles_m * a.tiles_n * a.B;
    if (a.n_tiles == 0) return TFB_OK;
    int grid = (int)std::min<int64_t>(a.n_tiles, (int64_t)ctx->sm_count * 8);
    LaunchScope ls(ctx, "contract_simt");
    switch (p.dtype) {
        case TFB_F32: contract_simt_kernel<float><<<grid, 256, 0, ctx->stream>>>(a); break;
        case TFB_F64: contract_simt_kernel<double><<<grid, 256, 0, ctx->stream>>>(a); break;
        case TFB_C32: contract_simt_kernel<float2><<<grid, 256, 0, ctx->stream>>>(a); break;
        case TFB_C64: contract_simt_kernel<double2><<<grid, 256, 0, ctx->stream>>>(a); break;
        default: return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", p.dtype);
    }
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}

// The same kernel over a non-Standard semiring (real types only): 1 MaxPlus, 2 MinPlus.
tfb_status contract_simt_semiring(tfb_ctx* ctx, const ContractProblem& p, int algebra) {
    if (p.dtype != TFB_F32 && p.dtype != TFB_F64)
        return fail(TFB_ERR_INVALID_ARGUMENT, "MaxPlus and MinPlus are defined for f32 and f64");
    if (p.mul) return fail(TFB_ERR_INVALID_ARGUMENT, "a fused multiplier is a Standard-algebra feature");
    DeviceGuard guard(ctx->device);
    std::shared_ptr<ContractTables> t;
    TFB_TRY(get_tables(ctx, p, &t));
    ContractArgs a;
    fill_args(p, *t, &a);
    a.tiles_m = (a.M + 63) / 64;
    a.tiles_n = (a.N + 63) / 64;
    a.n_tiles = a.tiles_m * a.tiles_n * a.B;
    if (a.n_tiles == 0) return TFB_OK;
    int grid = (int)std::min<int64_t>(a.n_tiles, (int64_t)ctx->sm_count * 8);
    LaunchScope ls(ctx, "contract_simt_semiring");
    if (p.dtype == TFB_F32 && algebra == 1) contract_simt_kernel<float, 1><<<grid, 256, 0, ctx->stream>>>(a);
    else if (p.dtype == TFB_F32 && algebra == 2) contract_simt_kernel<float, 2><<<grid, 256, 0, ctx->stream>>>(a);
    else if (p.dtype == TFB_F64 && algebra == 1) contract_simt_kernel<double, 1><<<grid, 256, 0, ctx->stream>>>(a);
    else if (p.dtype == TFB_F64 && algebra == 2) contract_simt_kernel<double, 2><<<grid, 256, 0, ctx->stream>>>(a);
    else return fail(TFB_ERR_INVALID_ARGUMENT, "unknown algebra %d", algebra);
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}

// ------------------------------------------------------------------ selection
tfb_status launch_contract(tfb_ctx* ctx, const ContractProblem& p, int force_kernel, const char** used) {
    DeviceGuard g(ctx->device);
    if (used) *used = "none";
    const int64_t M = p.M(), N = p.N(), K = p.K(), B = p.B();
    if (M == 0 || N == 0 || B == 0) return TFB_OK;  // empty output
    if (K == 0) {
        // Empty sum: C = beta * C.
        std::vector<Mode> modes;
        for (auto* grp : {&p.batch, &p.m, &p.n})
            for (auto& m : *grp) modes.push_back(Mode{m.extent, {m.s[2], 0, 0}});
        LoopNest nest;
        TFB_TRY(make_nest(modes, &nest));
        if (used) *used = "scale";
        return launch_scale(ctx, p.dtype, nest, p.c, p.beta);
    }
    int want = force_kernel != CK_AUTO ? force_kernel : env_int("TFB_FORCE_KERNEL", CK_AUTO);
    bool declined = false;
    if (want == CK_AUTO || want == CK_TCGEN05) {
        if (p.dtype == TFB_F32 || p.dtype == TFB_C32) {
            if (p.dtype == TFB_C32)
                TFB_TRY(contract_c32_embedded(ctx, p, &declined));
            else
                TFB_TRY(contract_tcgen05(ctx, p, &declined));
            if (!declined) {
                if (used) *used = "tcgen05_tf32x3";
                return TFB_OK;
            }
            if (want == CK_TCGEN05)
                return fail(TFB_ERR_INVALID_ARGUMENT, "tcgen05 kernel forced but it cannot stage this layout");
        } else if (want == CK_TCGEN05) {
            return fail(TFB_ERR_INVALID_ARGUMENT, "tcgen05 kernel forced but the dtype is not f32/c32");
        }
    }
    if (want == CK_AUTO || want == CK_DMMA || want == CK_DMMA4) {
        if (p.dtype == TFB_F64 || p.dtype == TFB_C64) {
            const bool four = want == CK_DMMA4 || env_int("TFB_C64_FOUR_PRODUCTS", 0) != 0;
            TFB_TRY(contract_dmma(ctx, p, &declined, four));
            if (!declined) {
                if (used) *used = "dmma_f64";
                return TFB_OK;
            }
        } else if (want == CK_DMMA || want == CK_DMMA4) {
            return fail(TFB_ERR_INVALID_ARGUMENT, "DMMA kernel forced but the dtype is not f64/c64");
        }
    }
    if (used) *used = "simt";
    return contract_simt(ctx, p);
}

}  // namespace tfb
