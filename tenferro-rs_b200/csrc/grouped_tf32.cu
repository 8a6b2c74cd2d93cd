// Grouped f32 products on the tensor cores (mma.sync): the fast path of tfb_grouped_gemm for ragged
// batches of small column-major problems (every dimension a multiple of 16, at most 128
// deep - e.g. 4096 problems with dims drawn from {16, 32, 64, 128}).
//
// Such a batch is bound by HBM and by latency (2.7 - 21 flop per byte, a few microseconds of
// work per problem), not by arithmetic, so the kernel is built around moving each operand once
// and never waiting for it:
//
//   * a unit of work is one 64 x 64 output tile of one problem; it runs as one or two STAGES
//     of at most 64 of its K each;
//   * the host lays out, once per table, the exact stage sequence of every CTA of the launch
//     (units sorted longest first and dealt round-robin, 48-byte records with pre-offset
//     pointers), so the device does no scheduling arithmetic and takes no atomics;
//   * a CTA double-buffers stages in shared memory: the panels of stage s + 1 (A: 64 x K',
//     B: K' x 64, 16-byte cp.async) are requested before stage s is computed, the record of
//     stage s + 2 is already in registers;
//   * warp-level m16n8k8 TF32 MMAs, the 3xTF32 split done on the fragments in registers with
//     integer operations; the four warps tile a unit as 2 x 2, 4 x 1 or 1 x 4 so that small
//     units keep all of them busy;
//   * the tile leaves from registers in whole 32-byte sectors.
// Three CTAs per SM; nothing ever waits on another CTA.
//
// The tcgen05 form of this kernel (grouped_tcgen05.cu) is slower on these tables - 96 us against
// 54 for 4096 problems - because 3xTF32 from shared memory is bound by shared-memory bandwidth
// and by the cost of issuing one MMA per 8 of K, and its 128-row tiles are mostly padding for
// 16 - 64 row problems; it takes the tables this kernel declines.
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
constexpr int GKS = 64;            // deepest stage
constexpr int LDA = GT + 4;        // [k][m] pitch: 8-byte fragment reads of a half-warp hit 32 distinct banks
constexpr int LDBPAD = 8;          // [n][k] pitch = K' + 8, for the same reason
constexpr int kThreads = 128;
constexpr int kCtasPerSm = 3;
constexpr int kStageFloats = GKS * LDA + GT * (GKS + LDBPAD);

enum : unsigned short { kFirst = 1 << 8, kLast = 1 << 9, kEnd = 1 << 10 };

// One stage of one unit, ready to run: pointers already moved to the tile's corner and to the
// stage's first k.  48 bytes.
struct __align__(16) Stage {
    const float* a;   // A[m, k] at a + m + k * a_cs
    const float* b;   // B[k, n] at b + k + n * b_cs
    float* c;         // C[m, n] at c + m + n * c_cs
    int a_cs, b_cs, c_cs;
    unsigned short mt, nt, k;
    // bits 0-1: log2(warp rows); 2-3: blocks of 16 rows per warp; 4-6: blocks of 8 columns per
    // warp; kFirst: clear the accumulators; kLast: store the tile; kEnd: no more stages.
    unsigned short shape;
};
static_assert(sizeof(Stage) == 48, "records are fetched as three 16-byte loads");

struct FastArgs {
    const Stage* stages;  // [row][cta]: row r of CTA c at stages[r * grid + c]; two kEnd rows close the table
    float alpha, beta;
};

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// 3xTF32 split without conversion instructions: the tensor core reads the upper 19 bits of an
// f32, so the raw word serves as the (truncated) big part; the remainder is exact in f32 and
// gets half a TF32 ulp added so that the hardware's truncation of it rounds instead.
__device__ __forceinline__ void split_tf32(float x, uint32_t& big, uint32_t& small) {
    big = __float_as_uint(x);
    small = __float_as_uint(x - __uint_as_float(big & 0xffffe000u)) + 0x1000u;
}
__device__ __forceinline__ float remainder_tf32(float x) {
    return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u);
}
// {lo, hi} as two bf16 in one register (lo in the lower half).
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// 16-byte chunks along the contiguous direction of each operand.  A power-of-two group of
// threads takes one row of the panel, so no thread divides.
__device__ __forceinline__ void load_panels(const Stage& u, float* As, float* Bs, int tid) {
    const int K = u.k, mt = u.mt, nt = u.nt, LDB = K + LDBPAD;
    const int mq = mt >> 2, kq = K >> 2;
    {
        const int tl = mq <= 4 ? 2 : mq <= 8 ? 3 : 4;
        const int x = tid & ((1 << tl) - 1), step = kThreads >> tl;
        if (x < mq)
            for (int k = tid >> tl; k < K; k += step)
                cp_async_16(As + k * LDA + 4 * x, u.a + (int64_t)k * u.a_cs + 4 * x, true);
    }
    {
        const int tl = kq <= 4 ? 2 : kq <= 8 ? 3 : 4;
        const int x = tid & ((1 << tl) - 1), step = kThreads >> tl;
        if (x < kq)
            for (int n = tid >> tl; n < nt; n += step)
                cp_async_16(Bs + n * LDB + 4 * x, u.b + (int64_t)n * u.b_cs + 4 * x, true);
    }
}

// The arithmetic of one CTA: place() fixes the warp's part of a unit, clear() zeroes the
// accumulators, stage() adds one stage's panels, store() writes the tile.

// Tensor cores.  The four warps tile the unit as 2 x 2, 4 x 1 or 1 x 4, each taking up to 2 blocks
// of 16 rows and up to 4 blocks of 8 columns: a 16 x 16 unit keeps two warps busy with one MMA
// shape each instead of one warp with eight.
// Fragment numbering: inside a 16-row block the MMA's rows g and g + 8 are rows 2g and 2g + 1 of
// the tile, and inside an 8-deep k-step its columns t and t + 4 are k = 2t and 2t + 1 (A and B
// agree, so the sum is the same).  Every fragment pair is then 8 contiguous bytes of a panel,
// and a thread's outputs pair up along m.
struct MmaPath {
    float acc[2][4][4], corr[2][4][4];
    int wm, wn;
    int ci, cj;  // live blocks of 16 rows (0..2) and of 8 columns (0..4) in this warp's part of the unit

    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][j][e] = corr[i][j][e] = 0.f;
    }
    __device__ __forceinline__ void place(const Stage& cur, int tid) {
        const int warp = tid >> 5;
        const int lw = cur.shape & 3, ni = (cur.shape >> 2) & 3, nj = (cur.shape >> 4) & 7;
        wm = (warp & ((1 << lw) - 1)) * 16 * ni;
        wn = (warp >> lw) * 8 * nj;
        ci = max(0, min(ni, (cur.mt - wm + 15) / 16));
        cj = max(0, min(nj, (cur.nt - wn + 7) / 8));
        if (ci == 0 || cj == 0) ci = cj = 0;
    }
    // One stage with NI x NJ blocks per warp, all live: the shapes are compile-time so that a small
    // unit issues only its own instructions (predicated-off ones still take issue slots).
    template <int NI, int NJ>
    __device__ __forceinline__ void stage_t(const Stage& cur, const float* As, const float* Bs, int tid) {
        const int lane = tid & 31, gq = lane >> 2, tq = lane & 3;
        const int K = cur.k, LDB = K + LDBPAD;
        const float* pa = As + (2 * tq) * LDA + wm + 2 * gq;
        const float* pb = Bs + (wn + gq) * LDB + 2 * tq;
#pragma unroll 2
        for (int k0 = 0; k0 < K; k0 += 8) {
            // Per 8-deep k-step and output block: one TF32 MMA for big x big and ONE bf16
            // m16n8k16 MMA for both corrections, its 16-deep K holding small_a x big_b in the
            // first eight positions and big_a x small_b in the other eight.  The corrections are
            // 2^-11 of the product, so bf16's 2^-9 rounding of them lands at 2^-20.
            uint32_t ab[NI][4], ac[NI][4], bb[NJ][2], bc[NJ][2];
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const float2 lo = *reinterpret_cast<const float2*>(pa + k0 * LDA + 16 * i);
                const float2 hi = *reinterpret_cast<const float2*>(pa + (k0 + 1) * LDA + 16 * i);
                ab[i][0] = __float_as_uint(lo.x); ab[i][1] = __float_as_uint(lo.y);
                ab[i][2] = __float_as_uint(hi.x); ab[i][3] = __float_as_uint(hi.y);
                ac[i][0] = pack_bf16(remainder_tf32(lo.x), remainder_tf32(hi.x));  // row g,     k 2t, 2t+1
                ac[i][1] = pack_bf16(remainder_tf32(lo.y), remainder_tf32(hi.y));  // row g + 8
                ac[i][2] = pack_bf16(lo.x, hi.x);                                  // row g,     k 8 + 2t, ...
                ac[i][3] = pack_bf16(lo.y, hi.y);                                  // row g + 8
            }
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const float2 v = *reinterpret_cast<const float2*>(pb + 8 * j * LDB + k0);
                bb[j][0] = __float_as_uint(v.x); bb[j][1] = __float_as_uint(v.y);
                bc[j][0] = pack_bf16(v.x, v.y);
                bc[j][1] = pack_bf16(remainder_tf32(v.x), remainder_tf32(v.y));
            }
#pragma unroll
            for (int i = 0; i < NI; ++i)
#pragma unroll
                for (int j = 0; j < NJ; ++j) mma_bf16(corr[i][j], ac[i], bc[j]);
#pragma unroll
            for (int i = 0; i < NI; ++i)
#pragma unroll
                for (int j = 0; j < NJ; ++j) mma_tf32(acc[i][j], ab[i], bb[j]);
        }
    }
    // A warp's store covers 64 contiguous bytes in each of 4 columns: whole sectors.
    template <int NI, int NJ>
    __device__ __forceinline__ void store_t(const Stage& cur, float alpha, float beta, int tid) {
        const int lane = tid & 31, gq = lane >> 2, tq = lane & 3;
        const bool read_c = beta != 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i)
#pragma unroll
            for (int j = 0; j < NJ; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int m = wm + 16 * i + 2 * gq, n = wn + 8 * j + 2 * tq + e;
                    float2* dst = reinterpret_cast<float2*>(cur.c + m + (int64_t)n * cur.c_cs);
                    float2 v = make_float2(alpha * (acc[i][j][e] + corr[i][j][e]),
                                           alpha * (acc[i][j][e + 2] + corr[i][j][e + 2]));
                    if (read_c) {
                        const float2 o = *dst;
                        v.x += beta * o.x;
                        v.y += beta * o.y;
                    }
                    *dst = v;
                }
    }
#define TFB_GROUPED_SHAPES(CALL)                                                  \
    switch (ci * 8 + cj) {                                                        \
        case 1 * 8 + 1: CALL(1, 1); break;                                        \
        case 1 * 8 + 2: CALL(1, 2); break;                                        \
        case 1 * 8 + 3: CALL(1, 3); break;                                        \
        case 1 * 8 + 4: CALL(1, 4); break;                                        \
        case 2 * 8 + 1: CALL(2, 1); break;                                        \
        case 2 * 8 + 2: CALL(2, 2); break;                                        \
        case 2 * 8 + 3: CALL(2, 3); break;                                        \
        case 2 * 8 + 4: CALL(2, 4); break;                                        \
        default: break; /* this warp has no part of the unit */                   \
    }
    __device__ __forceinline__ void stage(const Stage& cur, const float* As, const float* Bs, int tid) {
#define TFB_CALL(NI, NJ) stage_t<NI, NJ>(cur, As, Bs, tid)
        TFB_GROUPED_SHAPES(TFB_CALL)
#undef TFB_CALL
    }
    __device__ __forceinline__ void store(const Stage& cur, float alpha, float beta, int tid) {
#define TFB_CALL(NI, NJ) store_t<NI, NJ>(cur, alpha, beta, tid)
        TFB_GROUPED_SHAPES(TFB_CALL)
#undef TFB_CALL
    }
#undef TFB_GROUPED_SHAPES
};

template <typename Path>
__device__ __forceinline__ void run_cta(const FastArgs& g, float* smem) {
    const int tid = threadIdx.x;
    const Stage* table = g.stages + blockIdx.x;
    const size_t pitch = gridDim.x;
    Stage cur = table[0];
    if (cur.shape & kEnd) return;
    Stage nxt = table[pitch];
    load_panels(cur, smem, smem + GKS * LDA, tid);
    cp_async_commit();
    Path path;
    int buf = 0;
    for (size_t row = 2;; ++row) {
        const Stage after = table[row * pitch];  // lands while this stage computes
        const bool more = !(nxt.shape & kEnd);
        {
            float* nb = smem + (buf ^ 1) * kStageFloats;
            if (more) load_panels(nxt, nb, nb + GKS * LDA, tid);
            cp_async_commit();  // an empty group when there is nothing to load keeps the count below right
        }
        cp_async_wait<1>();  // everything but the group just committed: this stage's panels
        __syncthreads();
        const float* As = smem + buf * kStageFloats;  // [K'][LDA]    (m contiguous, as in memory)
        const float* Bs = As + GKS * LDA;             // [64][K' + 8] (k contiguous, as in memory)
        if (cur.shape & kFirst) {
            path.place(cur, tid);
            path.clear();
        }
        path.stage(cur, As, Bs, tid);
        if (cur.shape & kLast) path.store(cur, g.alpha, g.beta, tid);
        if (!more) break;
        __syncthreads();  // every warp is done with this buffer before the stage after next lands in it
        cur = nxt;
        nxt = after;
        buf ^= 1;
    }
}

template <typename Path>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) grouped_f32_kernel(FastArgs g) {
    extern __shared__ __align__(16) float smem[];
    run_cta<Path>(g, smem);
}

}  // namespace

// Builds the device-resident schedule of a table when every problem qualifies for the
// tensor-core kernel; otherwise *declined = true and nothing is allocated.
tfb_status grouped_tf32_prepare(tfb_ctx* ctx, size_t n, const tfb_gemm_problem* problems, GroupedFast* out,
                                bool* declined) {
    *declined = true;
    if (n == 0 || env_int("TFB_NO_GROUPED_TC", 0)) return TFB_OK;
    struct UnitRef {
        uint32_t problem;
        uint16_t m0, n0;
        int64_t cost;
    };
    std::vector<UnitRef> units;
    units.reserve(n * 2);
    for (size_t p = 0; p < n; ++p) {
        const auto& q = problems[p];
        const bool dims_ok = q.m > 0 && q.n > 0 && q.k > 0 && q.m % 16 == 0 && q.n % 16 == 0 && q.k % 16 == 0 &&
                             q.k <= GKMAX && q.m < 65536 && q.n < 65536;
        const bool layout_ok = q.a_rs == 1 && q.b_rs == 1 && q.c_rs == 1 && q.a_cs % 4 == 0 && q.b_cs % 4 == 0 &&
                               q.c_cs % 4 == 0 && q.a_cs >= q.m && q.b_cs >= q.k && q.c_cs >= q.m &&
                               q.a_cs < INT32_MAX && q.b_cs < INT32_MAX && q.c_cs < INT32_MAX;
        const bool align_ok = ((uintptr_t)q.a % 16 == 0) && ((uintptr_t)q.b % 16 == 0) && ((uintptr_t)q.c % 16 == 0);
        if (!dims_ok || !layout_ok || !align_ok || p > UINT32_MAX) return TFB_OK;
        for (int64_t n0 = 0; n0 < q.n; n0 += GT)
            for (int64_t m0 = 0; m0 < q.m; m0 += GT) {
                const int64_t mt = std::min<int64_t>(GT, q.m - m0), nt = std::min<int64_t>(GT, q.n - n0);
                units.push_back({(uint32_t)p, (uint16_t)m0, (uint16_t)n0, q.k * (mt + nt) + mt * nt});
            }
    }
    // Longest units first, dealt round-robin: CTA c takes units c, c + grid, c + 2 grid, ... - one
    // from every band of the sorted list, so the CTAs' totals come out close and the tail is
    // made of short units.
    std::stable_sort(units.begin(), units.end(), [](const UnitRef& x, const UnitRef& y) { return x.cost > y.cost; });
    const int grid = (int)std::min<size_t>(units.size(), (size_t)ctx->sm_count * kCtasPerSm);
    std::vector<std::vector<Stage>> per_cta(grid);
    for (size_t i = 0; i < units.size(); ++i) {
        const UnitRef& r = units[i];
        const auto& q = problems[r.problem];
        Stage s;
        s.a_cs = (int)q.a_cs; s.b_cs = (int)q.b_cs; s.c_cs = (int)q.c_cs;
        s.mt = (unsigned short)std::min<int64_t>(GT, q.m - r.m0);
        s.nt = (unsigned short)std::min<int64_t>(GT, q.n - r.n0);
        s.c = (float*)q.c + r.m0 + (int64_t)r.n0 * q.c_cs;
        // Warp grid with the fewest MMA shapes per warp; 2 x 2 always fits.
        const int rows16 = s.mt / 16, cols8 = s.nt / 8;
        int best_lw = 1, best_ni = (rows16 + 1) / 2, best_nj = (cols8 + 1) / 2;
        const int cand[2][2] = {{2, 4}, {0, 1}};  // {log2(warp rows), warp rows}
        for (const auto& cd : cand) {
            const int wr = cd[1], wc = 4 / wr;
            const int ni = (rows16 + wr - 1) / wr, nj = (cols8 + wc - 1) / wc;
            if (ni <= 2 && nj <= 4 && ni * nj < best_ni * best_nj) {
                best_lw = cd[0]; best_ni = ni; best_nj = nj;
            }
        }
        const unsigned short shape = (unsigned short)(best_lw | (best_ni << 2) | (best_nj << 4));
        for (int64_t k0 = 0; k0 < q.k; k0 += GKS) {
            s.a = (const float*)q.a + r.m0 + k0 * q.a_cs;
            s.b = (const float*)q.b + k0 + (int64_t)r.n0 * q.b_cs;
            s.k = (unsigned short)std::min<int64_t>(GKS, q.k - k0);
            s.shape = (unsigned short)(shape | (k0 == 0 ? kFirst : 0) | (k0 + GKS >= q.k ? kLast : 0));
            per_cta[i % grid].push_back(s);
        }
    }
    size_t rows = 0;
    for (const auto& v : per_cta) rows = std::max(rows, v.size());
    rows += 2;  // the kernel reads two records ahead
    Stage end_mark{};
    end_mark.shape = kEnd;
    std::vector<Stage> table(rows * (size_t)grid, end_mark);
    for (int c = 0; c < grid; ++c)
        for (size_t r = 0; r < per_cta[c].size(); ++r) table[r * grid + c] = per_cta[c][r];
    const size_t bytes = table.size() * sizeof(Stage);
    TFB_TRY(out->mem.alloc(ctx, bytes));
    // `table` is pageable: the copy has been staged by the time the call returns.
    TFB_CUDA(cudaMemcpyAsync(out->mem.ptr, table.data(), bytes, cudaMemcpyHostToDevice, ctx->stream));
    out->total_units = (int64_t)units.size();
    out->grid = grid;
    *declined = false;
    return TFB_OK;
}

tfb_status grouped_tf32_run(tfb_ctx* ctx, const GroupedFast& f, Scalar alpha, Scalar beta, bool* declined) {
    *declined = true;
    if (alpha.im != 0 || beta.im != 0) return TFB_OK;
    *declined = false;
    FastArgs g;
    g.stages = (const Stage*)f.mem.ptr;
    g.alpha = (float)alpha.re;
    g.beta = (float)beta.re;
    const int smem = 2 * kStageFloats * (int)sizeof(float);
    static std::mutex mu;
    static std::map<int, bool> configured;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[ctx->device]) {
            TFB_CUDA(cudaFuncSetAttribute(grouped_f32_kernel<MmaPath>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            configured[ctx->device] = true;
        }
    }
    LaunchScope ls(ctx, "grouped_tf32x3");
    grouped_f32_kernel<MmaPath><<<f.grid, kThreads, smem, ctx->stream>>>(g);
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}

}  // namespace tfb
