// f64 / Complex64 contraction on the FP64 tensor pipe (mma.sync m8n8k4 DMMA).
//
// tcgen05 has no f64 kind, so double precision runs on the warp-level DMMA instruction.
// Operand tiles are gathered from the strided tensors with cp.async through the offset
// tables (any strides; 16-byte chunks where the layout allows), kept in a multi-stage
// shared-memory ring, and consumed as m8n8k4 fragments.  Complex64 is four real DMMAs per
// fragment pair on interleaved (re, im) tiles; conjugation is a sign flip on the fragment.
//
// Work = (batch x M-tiles x N-tiles) x k-iterations, cut into equal contiguous ranges, one
// per CTA ("stream-K"): small outputs with long K (the 64 x 64 output of `abc,bcd->ad`, the
// 512 x 512 environments of an MPS transfer-matrix chain) still fill all SMs.  A range that
// cuts a tile writes its accumulators to a scratch slot; a second kernel adds the slots of
// each cut tile in a fixed order and applies alpha/beta, so results are reproducible run to
// run and no CTA ever waits for another.
//
// Semantics: PrimDescriptor::{Contract, BatchedGemm}, tenferro-prims/src/lib.rs:156-168,
// 227-239; execute contract :300-320.
#include "contract_common.cuh"
#include "contract_tables.h"

namespace tfb {

template <bool CPLX, int BM_, int BN_, int BK_, int WARPS_M_, int WARPS_N_, int STAGES_>
struct DmmaCfg {
    static constexpr bool kCplx = CPLX;
    static constexpr int BM = BM_, BN = BN_, BK = BK_, WARPS_M = WARPS_M_, WARPS_N = WARPS_N_, STAGES = STAGES_;
    static constexpr int NT = WARPS_M * WARPS_N * 32;
    static constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
    static constexpr int TM = WM / 8, TN = WN / 8;
    static constexpr int ES = CPLX ? 16 : 8;
    // Shared-memory pitches (elements).  K-fast tiles are [rows][PK]; M/N-fast tiles are
    // [BK][PM]/[BK][PN].  Pitches are chosen so that one fragment read of a half warp
    // (real, 8-byte) or quarter warp (complex, 16-byte) touches every bank once.
    static constexpr int PK = BK + 4;
    static constexpr int PM = BM + (CPLX ? 2 : 4);
    static constexpr int PN = BN + (CPLX ? 2 : 4);
    static constexpr int A_ELEMS = (BM * PK > BK * PM) ? BM * PK : BK * PM;
    static constexpr int B_ELEMS = (BN * PK > BK * PN) ? BN * PK : BK * PN;
    static constexpr int STAGE_BYTES = (A_ELEMS + B_ELEMS) * ES;
    static constexpr int SMEM_BYTES = STAGE_BYTES * STAGES;
    static constexpr int TILE_ELEMS = BM * BN;
};

__device__ __forceinline__ void dmma(double& c0, double& c1, double a, double b) {
    asm("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}

// Issue the cp.async gathers of one operand tile for k-iteration `kit`.
//   ROWS x BK elements; `fast_k` says whether threads (and chunks) run along k or along the row index.
//   row_tab / k_tab: offset tables; r0: first row of the tile; n_rows / K: bounds.
template <typename Cfg, int ROWS, int PROW, int VEC>
__device__ __forceinline__ void gather_tile(char* smem, const char* base, const int64_t* __restrict__ row_tab,
                                            const int64_t* __restrict__ k_tab, int64_t r0, int64_t n_rows, int64_t k0,
                                            int64_t K, bool fast_k, int tid) {
    constexpr int ES = Cfg::ES;
    constexpr int CHUNKS = ROWS * Cfg::BK / VEC;
    constexpr int PER_THREAD = (CHUNKS + Cfg::NT - 1) / Cfg::NT;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        int c = tid + i * Cfg::NT;
        if (CHUNKS % Cfg::NT != 0 && c >= CHUNKS) break;
        int r, k;
        if (fast_k) {
            constexpr int KC = Cfg::BK / VEC;
            k = (c % KC) * VEC;
            r = c / KC;
        } else {
            constexpr int RC = ROWS / VEC;
            r = (c % RC) * VEC;
            k = c / RC;
        }
        const bool valid = (r0 + r < n_rows) && (k0 + k < K);
        const char* src = base;
        if (valid) src = base + (row_tab[r0 + r] + k_tab[k0 + k]) * (int64_t)ES;
        char* dst = smem + (size_t)(fast_k ? (r * Cfg::PK + k) : (k * PROW + r)) * ES;
        if (ES * VEC == 16)
            cp_async_16(dst, src, valid);
        else
            cp_async_8(dst, src, valid);
    }
}

template <typename Cfg>
__global__ void __launch_bounds__(Cfg::NT) contract_dmma_kernel(ContractArgs g) {
    constexpr bool CPLX = Cfg::kCplx;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN, STAGES = Cfg::STAGES;
    constexpr int ES = Cfg::ES;
    extern __shared__ __align__(16) char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm0 = (warp % Cfg::WARPS_M) * Cfg::WM, wn0 = (warp / Cfg::WARPS_M) * Cfg::WN;
    const int lr = lane >> 2, lc = lane & 3;  // fragment row / k (or column pair)

    // Runtime element strides inside the shared tiles.
    const int a_sm = g.a_kfast ? Cfg::PK : 1, a_sk = g.a_kfast ? 1 : Cfg::PM;
    const int b_sn = g.b_kfast ? Cfg::PK : 1, b_sk = g.b_kfast ? 1 : Cfg::PN;
    const int a_frag = (wm0 + lr) * a_sm + lc * a_sk;
    const int b_frag = (wn0 + lr) * b_sn + lc * b_sk;

    const int64_t it_begin = (int64_t)blockIdx.x * g.iters_per_cta;
    const int64_t it_end = min(g.total_iters, it_begin + g.iters_per_cta);
    const int64_t first_tile = it_begin / g.k_iters;

    int64_t it = it_begin;
    while (it < it_end) {
        const int64_t tile = it / g.k_iters;
        const int64_t kb = it - tile * g.k_iters;
        const int64_t ke = min(g.k_iters, kb + (it_end - it));
        const int64_t tm = tile % g.tiles_m;
        const int64_t rest = tile / g.tiles_m;
        const int64_t tn = rest % g.tiles_n;
        const int64_t bb = rest / g.tiles_n;
        const int64_t m0 = tm * BM, n0 = tn * BN;
        const char* Ab = g.a + g.a_b[bb] * (int64_t)ES;
        const char* Bb = g.b + g.b_b[bb] * (int64_t)ES;

        double acc[TM][TN][CPLX ? 4 : 2];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int e = 0; e < (CPLX ? 4 : 2); ++e) acc[i][j][e] = 0.0;

        auto issue = [&](int64_t kit, int slot) {
            char* sa = smem + (size_t)slot * Cfg::STAGE_BYTES;
            char* sb = sa + (size_t)Cfg::A_ELEMS * ES;
            const int64_t k0 = kit * BK;
            if (!CPLX && g.a_vec == 2)
                gather_tile<Cfg, BM, Cfg::PM, 2>(sa, Ab, g.a_m, g.a_k, m0, g.M, k0, g.K, g.a_kfast, tid);
            else
                gather_tile<Cfg, BM, Cfg::PM, 1>(sa, Ab, g.a_m, g.a_k, m0, g.M, k0, g.K, g.a_kfast, tid);
            if (!CPLX && g.b_vec == 2)
                gather_tile<Cfg, BN, Cfg::PN, 2>(sb, Bb, g.b_n, g.b_k, n0, g.N, k0, g.K, g.b_kfast, tid);
            else
                gather_tile<Cfg, BN, Cfg::PN, 1>(sb, Bb, g.b_n, g.b_k, n0, g.N, k0, g.K, g.b_kfast, tid);
        };

        // Prologue: fill STAGES-1 slots.
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (kb + s < ke) issue(kb + s, s);
            cp_async_commit();
        }
        int slot = 0;
        for (int64_t kit = kb; kit < ke; ++kit) {
            cp_async_wait<STAGES - 2>();
            __syncthreads();
            {
                const int64_t nxt = kit + STAGES - 1;
                int ns = slot + STAGES - 1;
                if (ns >= STAGES) ns -= STAGES;
                if (nxt < ke) issue(nxt, ns);
                cp_async_commit();
            }
            const char* sa = smem + (size_t)slot * Cfg::STAGE_BYTES;
            const char* sb = sa + (size_t)Cfg::A_ELEMS * ES;
#pragma unroll
            for (int kk = 0; kk < BK; kk += 4) {
                if (CPLX) {
                    double ar[TM], ai[TM], nai[TM], br[TN], bi[TN];
#pragma unroll
                    for (int i = 0; i < TM; ++i) {
                        double2 v = *reinterpret_cast<const double2*>(sa + (size_t)(a_frag + 8 * i * a_sm + kk * a_sk) * 16);
                        ar[i] = v.x;
                        ai[i] = g.conj_a ? -v.y : v.y;
                        nai[i] = -ai[i];
                    }
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        double2 v = *reinterpret_cast<const double2*>(sb + (size_t)(b_frag + 8 * j * b_sn + kk * b_sk) * 16);
                        br[j] = v.x;
                        bi[j] = g.conj_b ? -v.y : v.y;
                    }
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) {
                            dmma(acc[i][j][0], acc[i][j][1], ar[i], br[j]);
                            dmma(acc[i][j][2], acc[i][j][3], ar[i], bi[j]);
                            dmma(acc[i][j][0], acc[i][j][1], nai[i], bi[j]);
                            dmma(acc[i][j][2], acc[i][j][3], ai[i], br[j]);
                        }
                } else {
                    double af[TM], bf[TN];
#pragma unroll
                    for (int i = 0; i < TM; ++i)
                        af[i] = *reinterpret_cast<const double*>(sa + (size_t)(a_frag + 8 * i * a_sm + kk * a_sk) * 8);
#pragma unroll
                    for (int j = 0; j < TN; ++j)
                        bf[j] = *reinterpret_cast<const double*>(sb + (size_t)(b_frag + 8 * j * b_sn + kk * b_sk) * 8);
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) dmma(acc[i][j][0], acc[i][j][1], af[i], bf[j]);
                }
            }
            if (++slot == STAGES) slot = 0;
        }
        cp_async_wait<0>();
        __syncthreads();  // every warp is done with the ring before the next range refills it

        const bool whole = (kb == 0 && ke == g.k_iters);
        if (whole) {
            char* Cb = g.c + g.c_b[bb] * (int64_t)ES;
            const bool read_c = g.beta_re != 0.0 || g.beta_im != 0.0;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int64_t n = n0 + wn0 + 8 * j + 2 * lc + e;
                    if (n >= g.N) continue;
                    const int64_t cn = g.c_n[n];
#pragma unroll
                    for (int i = 0; i < TM; ++i) {
                        const int64_t m = m0 + wm0 + 8 * i + lr;
                        if (m >= g.M) continue;
                        char* p = Cb + (g.c_m[m] + cn) * (int64_t)ES;
                        if (CPLX) {
                            const double xr = acc[i][j][e], xi = acc[i][j][2 + e];
                            double2 o;
                            o.x = g.alpha_re * xr - g.alpha_im * xi;
                            o.y = g.alpha_re * xi + g.alpha_im * xr;
                            if (read_c) {
                                const double2 old = *reinterpret_cast<const double2*>(p);
                                o.x += g.beta_re * old.x - g.beta_im * old.y;
                                o.y += g.beta_re * old.y + g.beta_im * old.x;
                            }
                            *reinterpret_cast<double2*>(p) = o;
                        } else {
                            double o = g.alpha_re * acc[i][j][e];
                            if (read_c) o += g.beta_re * *reinterpret_cast<const double*>(p);
                            *reinterpret_cast<double*>(p) = o;
                        }
                    }
                }
            }
        } else {
            const int64_t slot_id = 2 * (int64_t)blockIdx.x + (tile == first_tile ? 0 : 1);
            char* P = g.partial + (size_t)slot_id * Cfg::TILE_ELEMS * ES;
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int nl = wn0 + 8 * j + 2 * lc + e;
#pragma unroll
                    for (int i = 0; i < TM; ++i) {
                        const int ml = wm0 + 8 * i + lr;
                        char* p = P + ((size_t)nl * BM + ml) * ES;
                        if (CPLX)
                            *reinterpret_cast<double2*>(p) = make_double2(acc[i][j][e], acc[i][j][2 + e]);
                        else
                            *reinterpret_cast<double*>(p) = acc[i][j][e];
                    }
                }
        }
        it += ke - kb;
    }
}

// Adds the scratch slots of every cut tile in CTA order and applies alpha/beta.
template <typename Cfg>
__global__ void __launch_bounds__(256) contract_dmma_fixup_kernel(ContractArgs g) {
    constexpr bool CPLX = Cfg::kCplx;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, ES = Cfg::ES;
    const int64_t tile = blockIdx.x;
    const int64_t first_it = tile * g.k_iters, last_it = first_it + g.k_iters - 1;
    const int64_t g_first = first_it / g.iters_per_cta, g_last = last_it / g.iters_per_cta;
    if (g_first == g_last) return;  // one CTA held the whole tile and wrote it itself
    const int64_t tm = tile % g.tiles_m;
    const int64_t rest = tile / g.tiles_m;
    const int64_t tn = rest % g.tiles_n;
    const int64_t bb = rest / g.tiles_n;
    const int64_t m0 = tm * BM, n0 = tn * BN;
    char* Cb = g.c + g.c_b[bb] * (int64_t)ES;
    const bool read_c = g.beta_re != 0.0 || g.beta_im != 0.0;
    for (int idx = threadIdx.x; idx < BM * BN; idx += blockDim.x) {
        const int ml = idx % BM, nl = idx / BM;
        if (m0 + ml >= g.M || n0 + nl >= g.N) continue;
        double sr = 0.0, si = 0.0;
        for (int64_t c = g_first; c <= g_last; ++c) {
            const int64_t slot = 2 * c + (((c * g.iters_per_cta) / g.k_iters == tile) ? 0 : 1);
            const char* p = g.partial + ((size_t)slot * Cfg::TILE_ELEMS + idx) * ES;
            if (CPLX) {
                const double2 v = *reinterpret_cast<const double2*>(p);
                sr += v.x;
                si += v.y;
            } else {
                sr += *reinterpret_cast<const double*>(p);
            }
        }
        char* p = Cb + (g.c_m[m0 + ml] + g.c_n[n0 + nl]) * (int64_t)ES;
        if (CPLX) {
            double2 o;
            o.x = g.alpha_re * sr - g.alpha_im * si;
            o.y = g.alpha_re * si + g.alpha_im * sr;
            if (read_c) {
                const double2 old = *reinterpret_cast<const double2*>(p);
                o.x += g.beta_re * old.x - g.beta_im * old.y;
                o.y += g.beta_re * old.y + g.beta_im * old.x;
            }
            *reinterpret_cast<double2*>(p) = o;
        } else {
            double o = g.alpha_re * sr;
            if (read_c) o += g.beta_re * *reinterpret_cast<const double*>(p);
            *reinterpret_cast<double*>(p) = o;
        }
    }
}

template <typename Cfg>
static tfb_status run_cfg(tfb_ctx* ctx, const ContractProblem& p, ContractArgs a) {
    static std::mutex mu;
    static std::map<int, int> occupancy;  // per device
    int occ = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = occupancy.find(ctx->device);
        if (it == occupancy.end()) {
            TFB_CUDA(cudaFuncSetAttribute(contract_dmma_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          Cfg::SMEM_BYTES));
            TFB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, contract_dmma_kernel<Cfg>, Cfg::NT,
                                                                   Cfg::SMEM_BYTES));
            if (occ < 1) return fail(TFB_ERR_DEVICE, "DMMA kernel does not fit on an SM");
            occupancy[ctx->device] = occ;
        } else {
            occ = it->second;
        }
    }
    a.tiles_m = (a.M + Cfg::BM - 1) / Cfg::BM;
    a.tiles_n = (a.N + Cfg::BN - 1) / Cfg::BN;
    a.n_tiles = a.tiles_m * a.tiles_n * a.B;
    a.k_iters = (a.K + Cfg::BK - 1) / Cfg::BK;
    a.total_iters = a.n_tiles * a.k_iters;
    const int64_t slots = (int64_t)ctx->sm_count * occ;
    int64_t grid;
    if (a.n_tiles % slots == 0 || a.n_tiles >= 16 * slots) {
        // Whole tiles per CTA: nothing is cut.
        grid = std::min(a.n_tiles, slots);
        a.iters_per_cta = ((a.n_tiles + grid - 1) / grid) * a.k_iters;
    } else {
        // Equal shares of the iteration space, at least 4 k-iterations each.
        grid = std::min<int64_t>(slots, std::max<int64_t>(1, a.total_iters / 4));
        a.iters_per_cta = (a.total_iters + grid - 1) / grid;
    }
    grid = (a.total_iters + a.iters_per_cta - 1) / a.iters_per_cta;
    const bool cuts = a.iters_per_cta % a.k_iters != 0;
    PoolBlock ws;
    if (cuts) {
        TFB_TRY(ws.alloc(ctx, (size_t)grid * 2 * Cfg::TILE_ELEMS * Cfg::ES));
        a.partial = (char*)ws.ptr;
    }
    contract_dmma_kernel<Cfg><<<(unsigned)grid, Cfg::NT, Cfg::SMEM_BYTES, ctx->stream>>>(a);
    TFB_CUDA(cudaGetLastError());
    if (cuts) {
        contract_dmma_fixup_kernel<Cfg><<<(unsigned)a.n_tiles, 256, 0, ctx->stream>>>(a);
        TFB_CUDA(cudaGetLastError());
    }
    (void)p;
    return TFB_OK;
}

using RealBig = DmmaCfg<false, 128, 128, 16, 4, 4, 3>;
using RealSmall = DmmaCfg<false, 64, 64, 16, 2, 2, 4>;
using CplxMain = DmmaCfg<true, 64, 64, 8, 2, 4, 4>;
using CplxSmall = DmmaCfg<true, 32, 32, 8, 2, 2, 4>;

tfb_status contract_dmma(tfb_ctx* ctx, const ContractProblem& p, bool* declined) {
    *declined = false;
    if (p.dtype != TFB_F64 && p.dtype != TFB_C64) {
        *declined = true;
        return TFB_OK;
    }
    std::shared_ptr<ContractTables> t;
    TFB_TRY(get_tables(ctx, p, &t));
    ContractArgs a;
    fill_args(p, *t, &a);
    const int shape = env_int("TFB_DMMA_TILE", 0);  // 0 auto, 1 small, 2 big
    if (p.dtype == TFB_F64) {
        bool small = (a.M <= 64 || a.N <= 64 || a.M * a.N * a.B < (int64_t)128 * 128 * ctx->sm_count / 2);
        if (shape == 1) small = true;
        if (shape == 2) small = false;
        return small ? run_cfg<RealSmall>(ctx, p, a) : run_cfg<RealBig>(ctx, p, a);
    }
    bool small = (a.M <= 32 || a.N <= 32);
    if (shape == 1) small = true;
    if (shape == 2) small = false;
    return small ? run_cfg<CplxSmall>(ctx, p, a) : run_cfg<CplxMain>(ctx, p, a);
}

}  // namespace tfb
