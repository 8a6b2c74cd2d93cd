// f64 / Complex64 contraction on the FP64 tensor pipe (mma.sync DMMA).
//
// tcgen05 has no f64 kind, so double precision runs on the warp-level DMMA instruction
// (the m16n8k8 shape: it keeps the pipe fed with a quarter of the instructions of m8n8k4).
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

// m16n8k8: rows gid / gid + 8 of the 16-row tile, k = tig and tig + 4.
__device__ __forceinline__ void dmma16(double& c0, double& c1, double& c2, double& c3, double a0, double a1, double a2,
                                       double a3, double b0, double b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+d"(c0), "+d"(c1), "+d"(c2), "+d"(c3)
        : "d"(a0), "d"(a1), "d"(a2), "d"(a3), "d"(b0), "d"(b1));
}

// Offsets may be negative (reversed axes), so "outside the tensor" is a sentinel no real
// offset can take, not a sign.
constexpr int64_t kOutside = INT64_MIN;

// Per-thread state of the cp.async gather of one operand tile (ROWS x BK elements, VEC
// elements per chunk).  Row offsets are read from the table once per tile; the k offsets of
// the next k-iteration are fetched one iteration ahead, so no table load sits between a
// barrier and the copies that follow it.
template <typename Cfg, int ROWS, int PROW, int VEC>
struct Gather {
    static constexpr int ES = Cfg::ES;
    static constexpr int CHUNKS = ROWS * Cfg::BK / VEC;
    static constexpr int PT = (CHUNKS + Cfg::NT - 1) / Cfg::NT;
    int64_t row_off[PT];  // element offset of the chunk's row, or kOutside
    int64_t k_off[PT];    // element offset of the chunk's k for the prefetched iteration, or kOutside

    __device__ __forceinline__ static void coords(int c, bool fast_k, int& r, int& k) {
        if (fast_k) {
            constexpr int KC = Cfg::BK / VEC;
            k = (c % KC) * VEC;
            r = c / KC;
        } else {
            constexpr int RC = ROWS / VEC;
            r = (c % RC) * VEC;
            k = c / RC;
        }
    }
    __device__ __forceinline__ void set_tile(const int64_t* __restrict__ row_tab, int64_t r0, int64_t n_rows,
                                             bool fast_k, int tid) {
#pragma unroll
        for (int i = 0; i < PT; ++i) {
            const int c = tid + i * Cfg::NT;
            int r, k;
            coords(c, fast_k, r, k);
            row_off[i] = (c < CHUNKS && r0 + r < n_rows) ? __ldg(row_tab + r0 + r) : kOutside;
        }
    }
    __device__ __forceinline__ void prefetch(const int64_t* __restrict__ k_tab, int64_t k0, int64_t K, bool fast_k,
                                             int tid) {
#pragma unroll
        for (int i = 0; i < PT; ++i) {
            const int c = tid + i * Cfg::NT;
            int r, k;
            coords(c, fast_k, r, k);
            k_off[i] = (k0 + k < K) ? __ldg(k_tab + k0 + k) : kOutside;
        }
    }
    __device__ __forceinline__ void issue(char* smem, const char* base, bool fast_k, int tid) const {
#pragma unroll
        for (int i = 0; i < PT; ++i) {
            const int c = tid + i * Cfg::NT;
            if (CHUNKS % Cfg::NT != 0 && c >= CHUNKS) break;
            int r, k;
            coords(c, fast_k, r, k);
            const bool valid = row_off[i] != kOutside && k_off[i] != kOutside;
            const char* src = valid ? base + (row_off[i] + k_off[i]) * (int64_t)ES : base;
            char* dst = smem + (size_t)(fast_k ? (r * Cfg::PK + k) : (k * PROW + r)) * ES;
            if (ES * VEC == 16)
                cp_async_16(dst, src, valid);
            else
                cp_async_8(dst, src, valid);
        }
    }
};

template <typename Cfg, int VA, int VB>
__device__ __forceinline__ void dmma_range(const ContractArgs& g, char* smem, int64_t it_begin, int64_t it_end) {
    constexpr bool CPLX = Cfg::kCplx;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN, STAGES = Cfg::STAGES;
    constexpr int ES = Cfg::ES;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm0 = (warp % Cfg::WARPS_M) * Cfg::WM, wn0 = (warp / Cfg::WARPS_M) * Cfg::WN;
    const int lr = lane >> 2, lc = lane & 3;  // fragment row / k (or column pair)
    const bool a_kfast = g.a_kfast, b_kfast = g.b_kfast;

    // Runtime element strides inside the shared tiles.
    const int a_sm = a_kfast ? Cfg::PK : 1, a_sk = a_kfast ? 1 : Cfg::PM;
    const int b_sn = b_kfast ? Cfg::PK : 1, b_sk = b_kfast ? 1 : Cfg::PN;
    const int a_frag = (wm0 + lr) * a_sm + lc * a_sk;
    const int b_frag = (wn0 + lr) * b_sn + lc * b_sk;
    const int64_t first_tile = it_begin / g.k_iters;

    Gather<Cfg, BM, Cfg::PM, VA> ga;
    Gather<Cfg, BN, Cfg::PN, VB> gb;

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
        ga.set_tile(g.a_m, m0, g.M, a_kfast, tid);
        gb.set_tile(g.b_n, n0, g.N, b_kfast, tid);

        double acc[TM][TN][CPLX ? 4 : 2];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int e = 0; e < (CPLX ? 4 : 2); ++e) acc[i][j][e] = 0.0;

        // `fetch(kit)` loads the k offsets of iteration kit; `issue(slot)` starts its copies.
        auto fetch = [&](int64_t kit) {
            ga.prefetch(g.a_k, kit * BK, g.K, a_kfast, tid);
            gb.prefetch(g.b_k, kit * BK, g.K, b_kfast, tid);
        };
        auto issue = [&](int slot) {
            char* sa = smem + (size_t)slot * Cfg::STAGE_BYTES;
            char* sb = sa + (size_t)Cfg::A_ELEMS * ES;
            ga.issue(sa, Ab, a_kfast, tid);
            gb.issue(sb, Bb, b_kfast, tid);
        };

        // Prologue: fill STAGES-1 slots.
        fetch(kb);
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (kb + s < ke) {
                issue(s);
                fetch(kb + s + 1);
            }
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
                if (nxt < ke) {
                    issue(ns);
                    fetch(nxt + 1);
                }
                cp_async_commit();
            }
            const char* sa = smem + (size_t)slot * Cfg::STAGE_BYTES;
            const char* sb = sa + (size_t)Cfg::A_ELEMS * ES;
#pragma unroll
            for (int kk = 0; kk < BK; kk += 8) {
                // One m16n8k8 step: fragments of the two 8-row halves (h) and the two 4-deep
                // k halves (q) of every m16 tile; the 8-column tiles of B likewise.
                if (CPLX) {
                    double ar[TM][2], ai[TM][2], nai[TM][2], br[TN][2], bi[TN][2];
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            double2 v = *reinterpret_cast<const double2*>(
                                sa + (size_t)(a_frag + 8 * i * a_sm + (kk + 4 * q) * a_sk) * 16);
                            ar[i][q] = v.x;
                            ai[i][q] = g.conj_a ? -v.y : v.y;
                            nai[i][q] = -ai[i][q];
                        }
#pragma unroll
                    for (int j = 0; j < TN; ++j)
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            double2 v = *reinterpret_cast<const double2*>(
                                sb + (size_t)(b_frag + 8 * j * b_sn + (kk + 4 * q) * b_sk) * 16);
                            br[j][q] = v.x;
                            bi[j][q] = g.conj_b ? -v.y : v.y;
                        }
                    // Four passes over the warp tile; the two updates of one accumulator are
                    // (TM / 2) * TN * 2 instructions apart.
#pragma unroll
                    for (int i = 0; i < TM; i += 2)
#pragma unroll
                        for (int j = 0; j < TN; ++j)
                            dmma16(acc[i][j][0], acc[i][j][1], acc[i + 1][j][0], acc[i + 1][j][1], ar[i][0], ar[i + 1][0],
                                   ar[i][1], ar[i + 1][1], br[j][0], br[j][1]);
#pragma unroll
                    for (int i = 0; i < TM; i += 2)
#pragma unroll
                        for (int j = 0; j < TN; ++j)
                            dmma16(acc[i][j][2], acc[i][j][3], acc[i + 1][j][2], acc[i + 1][j][3], ar[i][0], ar[i + 1][0],
                                   ar[i][1], ar[i + 1][1], bi[j][0], bi[j][1]);
#pragma unroll
                    for (int i = 0; i < TM; i += 2)
#pragma unroll
                        for (int j = 0; j < TN; ++j)
                            dmma16(acc[i][j][0], acc[i][j][1], acc[i + 1][j][0], acc[i + 1][j][1], nai[i][0], nai[i + 1][0],
                                   nai[i][1], nai[i + 1][1], bi[j][0], bi[j][1]);
#pragma unroll
                    for (int i = 0; i < TM; i += 2)
#pragma unroll
                        for (int j = 0; j < TN; ++j)
                            dmma16(acc[i][j][2], acc[i][j][3], acc[i + 1][j][2], acc[i + 1][j][3], ai[i][0], ai[i + 1][0],
                                   ai[i][1], ai[i + 1][1], br[j][0], br[j][1]);
                } else {
                    double af[TM][2], bf[TN][2];
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int q = 0; q < 2; ++q)
                            af[i][q] = *reinterpret_cast<const double*>(
                                sa + (size_t)(a_frag + 8 * i * a_sm + (kk + 4 * q) * a_sk) * 8);
#pragma unroll
                    for (int j = 0; j < TN; ++j)
#pragma unroll
                        for (int q = 0; q < 2; ++q)
                            bf[j][q] = *reinterpret_cast<const double*>(
                                sb + (size_t)(b_frag + 8 * j * b_sn + (kk + 4 * q) * b_sk) * 8);
#pragma unroll
                    for (int i = 0; i < TM; i += 2)
#pragma unroll
                        for (int j = 0; j < TN; ++j)
                            dmma16(acc[i][j][0], acc[i][j][1], acc[i + 1][j][0], acc[i + 1][j][1], af[i][0], af[i + 1][0],
                                   af[i][1], af[i + 1][1], bf[j][0], bf[j][1]);
                }
            }
            if (++slot == STAGES) slot = 0;
        }
        cp_async_wait<0>();
        __syncthreads();  // every warp is done with the ring before the next range refills it

        const bool whole = (kb == 0 && ke == g.k_iters);
        if (whole) {
            if (g.mul) apply_mul_fragments<CPLX>(g, bb, m0 + wm0 + lr, n0 + wn0 + 2 * lc, acc);
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

template <typename Cfg>
__global__ void __launch_bounds__(Cfg::NT, 1) contract_dmma_kernel(ContractArgs g) {
    extern __shared__ __align__(16) char smem[];
    const int64_t it_begin = (int64_t)blockIdx.x * g.iters_per_cta;
    const int64_t it_end = min(g.total_iters, it_begin + g.iters_per_cta);
    if (Cfg::kCplx) {
        dmma_range<Cfg, 1, 1>(g, smem, it_begin, it_end);
    } else if (g.a_vec == 2 && g.b_vec == 2) {
        dmma_range<Cfg, 2, 2>(g, smem, it_begin, it_end);
    } else if (g.a_vec == 2) {
        dmma_range<Cfg, 2, 1>(g, smem, it_begin, it_end);
    } else if (g.b_vec == 2) {
        dmma_range<Cfg, 1, 2>(g, smem, it_begin, it_end);
    } else {
        dmma_range<Cfg, 1, 1>(g, smem, it_begin, it_end);
    }
}

// Adds the scratch slots of every cut tile in CTA order and applies alpha/beta.
// Grid: (tiles, kFixSplit); each CTA owns one slice of a tile's elements.
constexpr int kFixSplit = 4;
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
    constexpr int SLICE = BM * BN / kFixSplit;
    for (int idx = blockIdx.y * SLICE + threadIdx.x; idx < (blockIdx.y + 1) * SLICE; idx += blockDim.x) {
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
        if (g.mul) {
            const int64_t off = g.d_b[bb] + g.d_m[m0 + ml] + g.d_n[n0 + nl];
            if (CPLX) apply_mul_c128(g, off, sr, si);
            else apply_mul_f64(g, off, sr);
        }
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
            TFB_CUDA(cudaFuncSetAttribute(contract_dmma_kernel<Cfg>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
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
    {
        LaunchScope ls(ctx, "contract_dmma");
        contract_dmma_kernel<Cfg><<<(unsigned)grid, Cfg::NT, Cfg::SMEM_BYTES, ctx->stream>>>(a);
    }
    TFB_CUDA(cudaGetLastError());
    if (cuts) {
        LaunchScope ls(ctx, "contract_dmma_fixup");
        contract_dmma_fixup_kernel<Cfg><<<dim3((unsigned)a.n_tiles, kFixSplit), 256, 0, ctx->stream>>>(a);
        TFB_CUDA(cudaGetLastError());
    }
    (void)p;
    return TFB_OK;
}

}  // namespace tfb

#include "contract_dmma_tma.cuh"

namespace tfb {

using RealTma = DmmaTmaCfg<false, 128, 128, 16, 4, 4, 6>;
using CplxTma = DmmaTmaCfg<true, 64, 64, 16, 4, 4, 6>;
using RealTmaSmall = DmmaTmaCfg<false, 64, 64, 16, 2, 2, 8>;
using CplxTmaSmall = DmmaTmaCfg<true, 32, 32, 16, 2, 2, 8>;
using RealTmaTiny = DmmaTmaCfg<false, 32, 32, 16, 2, 2, 8>;
using RealBig = DmmaCfg<false, 128, 128, 16, 4, 4, 3>;
using RealBig8 = DmmaCfg<false, 128, 128, 16, 2, 4, 3>;
using RealSmall = DmmaCfg<false, 64, 64, 16, 2, 2, 4>;
using CplxMain = DmmaCfg<true, 64, 64, 16, 4, 4, 4>;
using CplxSmall = DmmaCfg<true, 32, 32, 8, 2, 2, 4>;

tfb_status contract_dmma(tfb_ctx* ctx, const ContractProblem& p, bool* declined, bool four_products) {
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
    const bool use_tma = !env_int("TFB_NO_DMMA_TMA", 0);
    if (p.dtype == TFB_F64) {
        bool small = (a.M <= 64 || a.N <= 64 || a.M * a.N * a.B < (int64_t)128 * 128 * ctx->sm_count / 2);
        if (shape == 1) small = true;
        if (shape == 2) small = false;
        if (shape == 3) return run_cfg<RealBig8>(ctx, p, a);
        if (use_tma) {
            bool d = true;
            if (a.M * a.N * a.B <= 64 * 64)
                TFB_TRY(run_tma_cfg<RealTmaTiny>(ctx, p, a, &d));  // few outputs, long K: many small ranges
            else if (small)
                TFB_TRY(run_tma_cfg<RealTmaSmall>(ctx, p, a, &d));
            else
                TFB_TRY(run_tma_cfg<RealTma>(ctx, p, a, &d));
            if (!d) return TFB_OK;
        }
        return small ? run_cfg<RealSmall>(ctx, p, a) : run_cfg<RealBig>(ctx, p, a);
    }
    bool small = (a.M <= 32 || a.N <= 32);
    if (shape == 1) small = true;
    if (shape == 2) small = false;
    // The TMA-fed kernel forms a complex product from three real ones, whose imaginary part is a
    // difference of sums as large as the real part: norm-wise exact, but when |Im| << |Re| the
    // imaginary part alone loses digits.  A caller that needs each part to its own accuracy asks
    // for four products, which the gather kernel below computes.
    if (use_tma && !four_products) {
        bool d = true;
        if (small)
            TFB_TRY(run_tma_cfg<CplxTmaSmall>(ctx, p, a, &d));
        else
            TFB_TRY(run_tma_cfg<CplxTma>(ctx, p, a, &d));
        if (!d) return TFB_OK;
    }
    return small ? run_cfg<CplxSmall>(ctx, p, a) : run_cfg<CplxMain>(ctx, p, a);
}

}  // namespace tfb
