// TMA-fed variant of the f64 / Complex64 DMMA contraction (included by contract_dmma.cu).
//
// When each of M, N, K is a single fused mode and one side of every operand has unit stride,
// the operand tiles need no per-thread gather: one thread issues two cp.async.bulk.tensor
// loads per k-iteration, a few iterations ahead, and the sixteen warps do nothing but
// fragment loads and DMMAs, synchronised by full/empty mbarriers (no CTA-wide barrier in
// the main loop, and the ring keeps running across the tiles of a stream-K range).
//
// The tensor maps are built so that the box lands in the order the m16n8k8 fragments are
// read, which makes every fragment load conflict-free without padding:
//   K-major operand   [k-panel of 4][row][4 k]     one 64-byte (complex) / 32-byte (real) run per row
//   MN-major operand  [row-group][k][G rows]       G = 2 (complex) or 4 (real): 32-byte runs
// (a quarter warp of 16-byte loads, or a half warp of 8-byte loads, then covers one
// contiguous 128-byte line).  Both are ordinary rank-4 tensor maps over the strided operand:
// dimension 0 is the short run, and a second dimension walks the same index in steps of the
// run length.
#pragma once
#include "ptx_sm100.cuh"

namespace tfb {

template <bool CPLX, int BM_, int BN_, int BK_, int WARPS_M_, int WARPS_N_, int STAGES_>
struct DmmaTmaCfg {
    using Base = DmmaCfg<CPLX, BM_, BN_, BK_, WARPS_M_, WARPS_N_, STAGES_>;  // tile shape, fix-up kernel
    static constexpr bool kCplx = CPLX;
    static constexpr int BM = BM_, BN = BN_, BK = BK_, WARPS_M = WARPS_M_, WARPS_N = WARPS_N_, STAGES = STAGES_;
    static constexpr int CONSUMERS = WARPS_M * WARPS_N;
    static constexpr int NT = CONSUMERS * 32;  // lane 0 of warp 0 doubles as the TMA producer
    static constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
    static constexpr int TM = WM / 8, TN = WN / 8;
    static constexpr int ES = CPLX ? 16 : 8;
    static constexpr int G = CPLX ? 2 : 4;  // rows per 32-byte run of an MN-major tile
    static constexpr int A_BYTES = BM * BK * ES, B_BYTES = BN * BK * ES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 16 * STAGES + 128;
};

// Element offset of (row, k) inside a dense tile.
template <typename Cfg, int ROWS, bool MN>
__device__ __forceinline__ int tile_off(int row, int k) {
    if (MN) return ((row / Cfg::G) * Cfg::BK + k) * Cfg::G + (row % Cfg::G);
    return ((k >> 2) * ROWS + row) * 4 + (k & 3);
}

template <typename Cfg, bool A_MN, bool B_MN>
__device__ __forceinline__ void dmma_tma_consume(const char* sa, const char* sb, double (&acc)[Cfg::TM][Cfg::TN][Cfg::kCplx ? 6 : 2],
                                                 int wm0, int wn0, int lr, int lc, bool conj_a, bool conj_b) {
    constexpr bool CPLX = Cfg::kCplx;
    constexpr int TM = Cfg::TM, TN = Cfg::TN;
#pragma unroll
    for (int kk = 0; kk < Cfg::BK; kk += 8) {
        if (CPLX) {
            // Three real products per complex one instead of four:
            //   P1 = Ar Br,  P2 = Ai Bi,  P3 = (Ar + Ai)(Br + Bi);  Re = P1 - P2,  Im = P3 - P1 - P2.
            // The sums cost two adds per fragment element; the FP64 pipe, which is what this
            // kernel waits for, issues a quarter fewer MMAs.  acc[..][0..1] = P1, [2..3] = P2,
            // [4..5] = P3; the caller folds them into Re / Im when a k range ends.
            double ar[TM][2], ai[TM][2], as[TM][2], br[TN][2], bi[TN][2], bs[TN][2];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const double2 v = *reinterpret_cast<const double2*>(
                        sa + (size_t)tile_off<Cfg, Cfg::BM, A_MN>(wm0 + 8 * i + lr, kk + 4 * q + lc) * 16);
                    ar[i][q] = v.x;
                    ai[i][q] = conj_a ? -v.y : v.y;
                    as[i][q] = ar[i][q] + ai[i][q];
                }
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const double2 v = *reinterpret_cast<const double2*>(
                        sb + (size_t)tile_off<Cfg, Cfg::BN, B_MN>(wn0 + 8 * j + lr, kk + 4 * q + lc) * 16);
                    br[j][q] = v.x;
                    bi[j][q] = conj_b ? -v.y : v.y;
                    bs[j][q] = br[j][q] + bi[j][q];
                }
#pragma unroll
            for (int i = 0; i < TM; i += 2)
#pragma unroll
                for (int j = 0; j < TN; ++j)
                    dmma16(acc[i][j][0], acc[i][j][1], acc[i + 1][j][0], acc[i + 1][j][1], ar[i][0], ar[i + 1][0], ar[i][1],
                           ar[i + 1][1], br[j][0], br[j][1]);
#pragma unroll
            for (int i = 0; i < TM; i += 2)
#pragma unroll
                for (int j = 0; j < TN; ++j)
                    dmma16(acc[i][j][2], acc[i][j][3], acc[i + 1][j][2], acc[i + 1][j][3], ai[i][0], ai[i + 1][0], ai[i][1],
                           ai[i + 1][1], bi[j][0], bi[j][1]);
#pragma unroll
            for (int i = 0; i < TM; i += 2)
#pragma unroll
                for (int j = 0; j < TN; ++j)
                    dmma16(acc[i][j][4], acc[i][j][5], acc[i + 1][j][4], acc[i + 1][j][5], as[i][0], as[i + 1][0], as[i][1],
                           as[i + 1][1], bs[j][0], bs[j][1]);
        } else {
            double af[TM][2], bf[TN][2];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    af[i][q] = *reinterpret_cast<const double*>(
                        sa + (size_t)tile_off<Cfg, Cfg::BM, A_MN>(wm0 + 8 * i + lr, kk + 4 * q + lc) * 8);
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    bf[j][q] = *reinterpret_cast<const double*>(
                        sb + (size_t)tile_off<Cfg, Cfg::BN, B_MN>(wn0 + 8 * j + lr, kk + 4 * q + lc) * 8);
#pragma unroll
            for (int i = 0; i < TM; i += 2)
#pragma unroll
                for (int j = 0; j < TN; ++j)
                    dmma16(acc[i][j][0], acc[i][j][1], acc[i + 1][j][0], acc[i + 1][j][1], af[i][0], af[i + 1][0], af[i][1],
                           af[i + 1][1], bf[j][0], bf[j][1]);
        }
    }
}

template <typename Cfg>
__global__ void __launch_bounds__(Cfg::NT, 1)
contract_dmma_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         ContractArgs g, int* status) {
    constexpr bool CPLX = Cfg::kCplx;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN, STAGES = Cfg::STAGES;
    constexpr int ES = Cfg::ES;
    extern __shared__ __align__(128) char smem_dyn[];
    char* smem = (char*)(((uintptr_t)smem_dyn + 127) & ~(uintptr_t)127);
    const uint32_t ring = smem_u32(smem);
    const uint32_t bars = ring + STAGES * Cfg::STAGE_BYTES;
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_empty = [&](int s) { return bars + 8u * (STAGES + s); };
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), Cfg::CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    } else if (tid == 32) {
        // the two descriptors travel while the barriers are being set up
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    __syncthreads();

    const int64_t it_begin = (int64_t)blockIdx.x * g.iters_per_cta;
    const int64_t it_end = min(g.total_iters, it_begin + g.iters_per_cta);
    const bool a_mn = !g.a_kfast, b_mn = !g.b_kfast;

    // ---------------------------------------------------------------- producer (lane 0 of warp 0)
    // It runs `kLead` k-iterations ahead of the consumers.  Issuing iteration j needs the slot
    // that iteration j - STAGES used, i.e. every warp must have finished that one; with
    // kLead = STAGES - 2 that is two iterations behind warp 0 itself, so the wait is short.
    constexpr int kLead = STAGES - 2;
    const int64_t my_iters = it_end - it_begin;
    int64_t issued = 0;
    // Position of the next k-iteration to issue, advanced without divisions: the producer is also a
    // computing thread, and whatever it spends here its whole warp waits for.  (32-bit: the host
    // keeps total_iters below 2^31 for this kernel.)
    uint32_t p_kit, p_tm, p_tn, p_bb;
    {
        const uint32_t k_iters = (uint32_t)g.k_iters, tiles_m = (uint32_t)g.tiles_m, tiles_n = (uint32_t)g.tiles_n;
        const uint32_t tile = (uint32_t)it_begin / k_iters, rest = tile / tiles_m;
        p_kit = (uint32_t)it_begin - tile * k_iters;
        p_tm = tile - rest * tiles_m;
        p_bb = rest / tiles_n;
        p_tn = rest - p_bb * tiles_n;
    }
    auto produce_until = [&](int64_t target) {
        if (target > my_iters) target = my_iters;
        for (; issued < target; ++issued) {
            const int m0 = (int)(p_tm * BM), n0 = (int)(p_tn * BN), k0 = (int)(p_kit * BK);
            const uint32_t bb = p_bb;
            const uint32_t iu = (uint32_t)issued;
            const int s = (int)(iu % STAGES);
            mbar_wait(bar_empty(s), ((iu / STAGES) & 1) ^ 1, status, 0x301);
            const uint32_t a_dst = ring + s * Cfg::STAGE_BYTES, b_dst = a_dst + Cfg::A_BYTES;
            mbar_expect_tx(bar_full(s), Cfg::STAGE_BYTES);
            if (a_mn) tma_load_4d(a_dst, &map_a, bar_full(s), 0, k0, m0 / Cfg::G, (int)bb);
            else      tma_load_4d(a_dst, &map_a, bar_full(s), 0, m0, k0 / 4, (int)bb);
            if (b_mn) tma_load_4d(b_dst, &map_b, bar_full(s), 0, k0, n0 / Cfg::G, (int)bb);
            else      tma_load_4d(b_dst, &map_b, bar_full(s), 0, n0, k0 / 4, (int)bb);
            if (++p_kit == (uint32_t)g.k_iters) {
                p_kit = 0;
                if (++p_tm == (uint32_t)g.tiles_m) {
                    p_tm = 0;
                    if (++p_tn == (uint32_t)g.tiles_n) {
                        p_tn = 0;
                        ++p_bb;
                    }
                }
            }
        }
    };
    const bool is_producer = (tid == 0);
    if (is_producer) produce_until(kLead);

    // -------------------------------------------------------------------- consumers
    const int wm0 = (warp % Cfg::WARPS_M) * Cfg::WM, wn0 = (warp / Cfg::WARPS_M) * Cfg::WN;
    const int lr = lane >> 2, lc = lane & 3;
    const bool conj_a = g.conj_a != 0, conj_b = g.conj_b != 0;
    uint32_t n = 0;
    int64_t it = it_begin;
    while (it < it_end) {
        const int64_t tile = it / g.k_iters;
        const int64_t kb = it - tile * g.k_iters;
        const int64_t ke = min(g.k_iters, kb + (it_end - it));
        const int64_t tm = tile % g.tiles_m, rest = tile / g.tiles_m, tn = rest % g.tiles_n, bb = rest / g.tiles_n;
        const int64_t m0 = tm * BM, n0 = tn * BN;
        double acc[TM][TN][CPLX ? 6 : 2];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j)
#pragma unroll
                for (int e = 0; e < (CPLX ? 6 : 2); ++e) acc[i][j][e] = 0.0;

        for (int64_t kit = kb; kit < ke; ++kit, ++n) {
            const int s = n % STAGES;
            if (is_producer) produce_until((int64_t)n + kLead + 1);
            if (lane == 0) mbar_wait(bar_full(s), (n / STAGES) & 1, status, 0x302);
            __syncwarp();
            const char* sa = smem + (size_t)s * Cfg::STAGE_BYTES;
            const char* sb = sa + Cfg::A_BYTES;
            if (a_mn) {
                if (b_mn) dmma_tma_consume<Cfg, true, true>(sa, sb, acc, wm0, wn0, lr, lc, conj_a, conj_b);
                else      dmma_tma_consume<Cfg, true, false>(sa, sb, acc, wm0, wn0, lr, lc, conj_a, conj_b);
            } else {
                if (b_mn) dmma_tma_consume<Cfg, false, true>(sa, sb, acc, wm0, wn0, lr, lc, conj_a, conj_b);
                else      dmma_tma_consume<Cfg, false, false>(sa, sb, acc, wm0, wn0, lr, lc, conj_a, conj_b);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(s));
        }

        if constexpr (CPLX) {
            // fold the three products of this k range into Re (slots 0-1) and Im (slots 2-3)
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const double p1 = acc[i][j][e], p2 = acc[i][j][2 + e], p3 = acc[i][j][4 + e];
                        acc[i][j][e] = p1 - p2;
                        acc[i][j][2 + e] = p3 - p1 - p2;
                    }
        }
        // A range that starts inside a tile (kb > 0) only contributes: it parks its
        // accumulators in this CTA's scratch slot and raises the CTA's flag.  The range that
        // holds the tile's first k-iteration owns the tile: it collects the contributions of
        // the CTAs after it, in CTA order, and writes C.  Contributions are the first thing a
        // CTA does and collecting is the last, so owners rarely wait; the wait is bounded.
        if (kb > 0 || g.sk_two_phase) {
            char* P = g.partial + (size_t)blockIdx.x * (BM * BN) * ES;
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        char* q = P + ((size_t)((i * TN + j) * 2 + e) * Cfg::NT + tid) * ES;
                        if (CPLX)
                            *reinterpret_cast<double2*>(q) = make_double2(acc[i][j][e], acc[i][j][2 + e]);
                        else
                            *reinterpret_cast<double*>(q) = acc[i][j][e];
                    }
            if (!g.sk_two_phase) {
                __threadfence();
                __syncthreads();
                if (tid == 0)
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.sk_flags + blockIdx.x), "r"(g.sk_epoch) : "memory");
            }
        } else {
            if (ke < g.k_iters) {
                const int64_t g_last = ((tile + 1) * g.k_iters - 1) / g.iters_per_cta;
                // All contributors' flags first (thread c - first polls flag c, bounded), then one
                // pass over their slots in CTA order: the loads of different slots overlap, the
                // additions keep their order, so the sum does not depend on timing.
                {
                    const int64_t c = (int64_t)blockIdx.x + 1 + tid;
                    if (c <= g_last) {
                        uint32_t v = 0;
                        for (uint32_t spin = 0; spin < (1u << 20); ++spin) {
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(g.sk_flags + c) : "memory");
                            if (v == g.sk_epoch) break;
                            __nanosleep(64);
                        }
                        if (v != g.sk_epoch) atomicCAS(status, 0, 0x303);
                    }
                    __syncthreads();
                }
#pragma unroll 4
                for (int64_t c = (int64_t)blockIdx.x + 1; c <= g_last; ++c) {
                    const char* P = g.partial + (size_t)c * (BM * BN) * ES;
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const char* q = P + ((size_t)((i * TN + j) * 2 + e) * Cfg::NT + tid) * ES;
                                if (CPLX) {
                                    const double2 v = __ldcg(reinterpret_cast<const double2*>(q));
                                    acc[i][j][e] += v.x;
                                    acc[i][j][2 + e] += v.y;
                                } else {
                                    acc[i][j][e] += __ldcg(reinterpret_cast<const double*>(q));
                                }
                            }
                }
            }
            if (g.mul) apply_mul_fragments<CPLX>(g, bb, m0 + wm0 + lr, n0 + wn0 + 2 * lc, acc);
            char* Cb = g.c + g.c_b[bb] * (int64_t)ES;
            const bool read_c = g.beta_re != 0.0 || g.beta_im != 0.0;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int64_t nn = n0 + wn0 + 8 * j + 2 * lc + e;
                    if (nn >= g.N) continue;
                    const int64_t cn = g.c_n[nn];
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
        }
        it += ke - kb;
    }
}

// Second phase of the two-launch split over K (outputs of a few tiles with a long K, such as
// 'abc,bcd->ad' with 64 x 64 outputs and K = 4096): every CTA of the main kernel has parked the
// sums of its k range in its slot; here one block per (tile, fragment) adds the `pieces` slots of
// a tile - one value per piece and thread, all loads independent, always in piece order, so the
// result does not depend on timing - and applies multiplier, alpha and beta.  The thread-to-element
// map is the main kernel's.  No CTA ever waits for another one.
template <typename Cfg>
__global__ void __launch_bounds__(Cfg::NT) dmma_tma_splitk_finish_kernel(ContractArgs g, int pieces) {
    constexpr bool CPLX = Cfg::kCplx;
    constexpr int BM = Cfg::BM, BN = Cfg::BN, TN = Cfg::TN, ES = Cfg::ES;
    const int64_t tile = blockIdx.x;
    const int f = blockIdx.y, i = f / (2 * TN), j = (f >> 1) % TN, e = f & 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t tm = tile % g.tiles_m, rest = tile / g.tiles_m, tn = rest % g.tiles_n, bb = rest / g.tiles_n;
    const int64_t m = tm * BM + (warp % Cfg::WARPS_M) * Cfg::WM + 8 * i + (lane >> 2);
    const int64_t n = tn * BN + (warp / Cfg::WARPS_M) * Cfg::WN + 8 * j + 2 * (lane & 3) + e;
    const char* P = g.partial + ((size_t)tile * pieces * (BM * BN) + (size_t)f * Cfg::NT + tid) * ES;
    double xr = 0.0, xi = 0.0;
#pragma unroll 8
    for (int s = 0; s < pieces; ++s) {
        const char* q = P + (size_t)s * (BM * BN) * ES;
        if (CPLX) {
            const double2 v = __ldcg(reinterpret_cast<const double2*>(q));
            xr += v.x;
            xi += v.y;
        } else {
            xr += __ldcg(reinterpret_cast<const double*>(q));
        }
    }
    if (m >= g.M || n >= g.N) return;
    if (g.mul) {
        const int64_t off = g.d_b[bb] + g.d_m[m] + g.d_n[n];
        if (CPLX) apply_mul_c128(g, off, xr, xi);
        else apply_mul_f64(g, off, xr);
    }
    char* p = g.c + (g.c_b[bb] + g.c_m[m] + g.c_n[n]) * (int64_t)ES;
    const bool read_c = g.beta_re != 0.0 || g.beta_im != 0.0;
    if (CPLX) {
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
        double o = g.alpha_re * xr;
        if (read_c) o += g.beta_re * *reinterpret_cast<const double*>(p);
        *reinterpret_cast<double*>(p) = o;
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledF64)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledF64 encode_tiled_f64() {
    static EncodeTiledF64 fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledF64)p;
    }();
    return fn;
}

// Tensor map of one operand (free group `fr`, tensor index tns); false when TMA cannot describe it.
template <typename Cfg>
static bool make_f64_map(const ContractProblem& p, const std::vector<Mode>& fr, int tns, const void* base, int rows,
                         bool* mn_major, CUtensorMap* map) {
    EncodeTiledF64 enc = encode_tiled_f64();
    if (!enc || fr.size() > 1 || p.k.size() != 1 || p.batch.size() > 1) return false;
    constexpr int W = Cfg::kCplx ? 2 : 1;  // doubles per element
    const int64_t R = fr.empty() ? 1 : fr[0].extent, rs = fr.empty() ? 0 : fr[0].s[tns];
    const int64_t K = p.k[0].extent, ks = p.k[0].s[tns];
    const int64_t B = p.batch.empty() ? 1 : p.batch[0].extent, bs = p.batch.empty() ? 0 : p.batch[0].s[tns];
    if ((uintptr_t)base % 16 != 0) return false;
    auto ok16 = [&](int64_t s) { return s > 0 && (s * W * 8) % 16 == 0; };
    if (B > 1 && !ok16(bs)) return false;
    cuuint64_t dims[4], strides[3];
    cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
    const cuuint64_t bstride = (cuuint64_t)((B > 1 ? bs * W * 8 : 16));
    if (ks == 1 && K % 4 == 0 && (R == 1 || ok16(rs))) {
        *mn_major = false;
        dims[0] = 4 * W; dims[1] = (cuuint64_t)R; dims[2] = (cuuint64_t)(K / 4); dims[3] = (cuuint64_t)B;
        strides[0] = (cuuint64_t)((R == 1 ? K : rs) * W * 8);
        strides[1] = 4 * W * 8;
        strides[2] = bstride;
        box[0] = 4 * W; box[1] = (cuuint32_t)rows; box[2] = Cfg::BK / 4; box[3] = 1;
    } else if (rs == 1 && R % Cfg::G == 0 && R > 1 && (K == 1 || ok16(ks))) {
        *mn_major = true;
        dims[0] = Cfg::G * W; dims[1] = (cuuint64_t)K; dims[2] = (cuuint64_t)(R / Cfg::G); dims[3] = (cuuint64_t)B;
        strides[0] = (cuuint64_t)((K == 1 ? R : ks) * W * 8);
        strides[1] = Cfg::G * W * 8;
        strides[2] = bstride;
        box[0] = Cfg::G * W; box[1] = Cfg::BK; box[2] = (cuuint32_t)(rows / Cfg::G); box[3] = 1;
    } else {
        return false;
    }
    for (int i = 0; i < 3; ++i)
        if (strides[i] % 16 != 0 || strides[i] >= (1ull << 40)) return false;
    for (int i = 0; i < 4; ++i)
        if (dims[i] == 0 || dims[i] > 0xffffffffull) return false;
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 4, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Runs the TMA-fed kernel when both operands qualify; otherwise *declined = true.
template <typename Cfg>
static tfb_status run_tma_cfg(tfb_ctx* ctx, const ContractProblem& p, ContractArgs a, bool* declined) {
    using Base = typename Cfg::Base;
    *declined = true;
    if (a.M > INT32_MAX - 512 || a.N > INT32_MAX - 512 || a.K > INT32_MAX - 64) return TFB_OK;
    CUtensorMap map_a, map_b;
    bool a_mn = false, b_mn = false;
    if (!make_f64_map<Cfg>(p, p.m, 0, p.a, Cfg::BM, &a_mn, &map_a)) return TFB_OK;
    if (!make_f64_map<Cfg>(p, p.n, 1, p.b, Cfg::BN, &b_mn, &map_b)) return TFB_OK;
    a.a_kfast = !a_mn;
    a.b_kfast = !b_mn;
    static std::mutex mu;
    static std::map<int, bool> configured;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[ctx->device]) {
            TFB_CUDA(cudaFuncSetAttribute(contract_dmma_tma_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          Cfg::SMEM_BYTES));
            configured[ctx->device] = true;
        }
    }
    a.tiles_m = (a.M + Cfg::BM - 1) / Cfg::BM;
    a.tiles_n = (a.N + Cfg::BN - 1) / Cfg::BN;
    a.n_tiles = a.tiles_m * a.tiles_n * a.B;
    a.k_iters = (a.K + Cfg::BK - 1) / Cfg::BK;
    a.total_iters = a.n_tiles * a.k_iters;
    if (a.total_iters >= ((int64_t)1 << 31)) return TFB_OK;  // the producer indexes k-iterations with 32 bits
    const int64_t slots = ctx->sm_count;  // one CTA per SM
    int64_t grid;
    // A handful of tiles with a long K: cut every tile into the same number of k pieces, one CTA
    // each, and add the pieces in a second, tiny launch.  (In the single-launch form below the
    // owner of a tile reads all its pieces itself - eight dependent round trips to L2 for 32
    // pieces - and 'abc,bcd->ad' at 64^4 took 16.4 us; here every load of the sum is independent.)
    int pieces = 0;
    if (a.n_tiles * 4 <= slots && a.k_iters >= 16 && env_int("TFB_SK_TWO_PHASE", 1)) {
        const int64_t want = std::min<int64_t>(std::min<int64_t>(32, slots / a.n_tiles), a.k_iters / 4);
        a.iters_per_cta = (a.k_iters + want - 1) / want;
        pieces = (int)((a.k_iters + a.iters_per_cta - 1) / a.iters_per_cta);
    }
    if (pieces > 1) {
        // ranges are per tile: CTA c takes piece c % pieces of tile c / pieces
        if (a.iters_per_cta * pieces != a.k_iters) {
            // the kernel cuts the linear (tile, k) space into equal ranges: pieces must divide K's iterations
            pieces = 0;
        }
    }
    if (pieces > 1) {
        grid = a.n_tiles * pieces;
        a.sk_two_phase = 1;
    } else if (a.n_tiles % slots == 0 || a.n_tiles >= 16 * slots) {
        grid = std::min(a.n_tiles, slots);
        a.iters_per_cta = ((a.n_tiles + grid - 1) / grid) * a.k_iters;
    } else {
        grid = std::min<int64_t>(slots, std::max<int64_t>(1, a.total_iters / 4));
        a.iters_per_cta = (a.total_iters + grid - 1) / grid;
        // One thread of the owner polls each contributor's flag and every contribution costs the
        // owner one pass over a slot: keep a tile in at most 32 pieces.
        a.iters_per_cta = std::max<int64_t>(a.iters_per_cta, (a.k_iters + 31) / 32);
    }
    if (!a.sk_two_phase) grid = (a.total_iters + a.iters_per_cta - 1) / a.iters_per_cta;
    const bool cuts = a.iters_per_cta % a.k_iters != 0;
    if (cuts) {
        // Scratch slots and flags live with the context (one slot per CTA, reused by every
        // launch; a flag is "raised" when it equals the launch's epoch, so nothing is reset).
        const size_t need = (size_t)grid * Base::TILE_ELEMS * Base::ES;
        if (ctx->sk_partial_bytes < need) {
            if (ctx->sk_partial) TFB_CUDA(cudaFree(ctx->sk_partial));
            ctx->sk_partial = nullptr;
            ctx->sk_partial_bytes = 0;
            TFB_CUDA(cudaMalloc(&ctx->sk_partial, need));
            ctx->sk_partial_bytes = need;
        }
        if (ctx->sk_flags_n < (size_t)grid) {
            if (ctx->sk_flags) TFB_CUDA(cudaFree(ctx->sk_flags));
            ctx->sk_flags = nullptr;
            ctx->sk_flags_n = 0;
            const size_t n = std::max<size_t>((size_t)grid, 1024);
            TFB_CUDA(cudaMalloc(&ctx->sk_flags, n * sizeof(unsigned)));
            TFB_CUDA(cudaMemset(ctx->sk_flags, 0, n * sizeof(unsigned)));
            ctx->sk_flags_n = n;
        }
        a.partial = (char*)ctx->sk_partial;
        a.sk_flags = ctx->sk_flags;
        if (ctx->capturing) {
            // A replayed launch would meet the flags its last run raised: a captured launch clears
            // them first and uses an epoch no live launch has.
            TFB_CUDA(cudaMemsetAsync(ctx->sk_flags, 0, (size_t)grid * sizeof(unsigned), ctx->stream));
            a.sk_epoch = 0xffffffffu;
        } else {
            a.sk_epoch = ++ctx->sk_epoch;
            if (a.sk_epoch == 0xffffffffu) a.sk_epoch = ctx->sk_epoch = 1;
        }
    }
    {
        LaunchScope ls(ctx, "contract_dmma");
        int* status = ctx->dev_status;
        void* args[] = {(void*)&map_a, (void*)&map_b, (void*)&a, (void*)&status};
        // Owners wait for contributors, so every CTA of the grid has to be resident: a
        // cooperative launch makes the runtime check that (grid <= one CTA per SM).
        if (cuts && !a.sk_two_phase && env_int("TFB_SK_COOP", 1))
            TFB_CUDA(cudaLaunchCooperativeKernel((const void*)contract_dmma_tma_kernel<Cfg>, dim3((unsigned)grid),
                                                 dim3(Cfg::NT), args, Cfg::SMEM_BYTES, ctx->stream));
        else
            contract_dmma_tma_kernel<Cfg><<<(unsigned)grid, Cfg::NT, Cfg::SMEM_BYTES, ctx->stream>>>(map_a, map_b, a, status);
    }
    TFB_CUDA(cudaGetLastError());
    if (a.sk_two_phase) {
        LaunchScope ls(ctx, "contract_dmma_finish");
        dmma_tma_splitk_finish_kernel<Cfg><<<dim3((unsigned)a.n_tiles, Cfg::TM * Cfg::TN * 2), Cfg::NT, 0, ctx->stream>>>(a, pieces);
        TFB_CUDA(cudaGetLastError());
    }
    *declined = false;
    return TFB_OK;
}

}  // namespace tfb
