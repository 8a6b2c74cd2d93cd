// f32 contraction on the 5th-generation tensor cores: TMA -> swizzled shared memory ->
// 3xTF32 split -> tcgen05.mma (kind::tf32) into a TMEM accumulator -> epilogue.
//
// Two kernels share the scheme.  The CTA-pair kernel (further down) is the one large outputs
// run on; the single-CTA kernel described first takes outputs with fewer than 129 rows or 256
// columns.  One CTA computes one 128 x BN tile of C (BN = 256 or 128).  Warp roles:
//   warp 0      TMA producer: one thread issues cp.async.bulk.tensor loads of the raw f32
//               operand tiles straight from the strided tensors (the "permute" of
//               permute-into-GEMM is the tensor map), 128-byte swizzle, zero fill at the edges;
//   warps 2-9   split every element: the raw word serves as the truncated big part (the tensor
//               core reads only its upper 19 bits); small = a - trunc(a), rounded to TF32, goes
//               to a second tile at the same swizzled position;
//   warp 1      one thread issues, per 8-deep k step, the three products
//               small*big, big*small, big*big into the same TMEM accumulator - f32 accuracy
//               from TF32 tensor cores (the dropped small*small term is ~2^-22 relative);
//   warps 2-9   promotion: every 8 k-blocks tcgen05.ld the finished work accumulator and add
//               it to an f32 running sum in registers (two work accumulators alternate, so
//               the tensor core never waits); epilogue: alpha/beta, store through the C
//               offset tables (any output strides).
// Stages cycle through mbarriers: full (TMA bytes landed) -> split (converters done) ->
// empty (tcgen05.commit: the MMAs that read the stage have retired); work accumulators
// through chunk_done (commit) -> promoted.  Every wait has an
// iteration bound; when one expires the kernel records a status word, keeps going with
// whatever data it has, frees its TMEM and returns - the host reports DeviceError.
//
// Operands may be K-major (contracted group has unit stride) or MN-major (free group has
// unit stride); the instruction descriptor's major bits select the layout, so neither needs
// a transpose pass.  Layouts TMA cannot describe (unit stride in neither group, strides that
// are not multiples of 16 bytes, more than two non-fusable modes per group) are repacked
// K-major first when the product is large, and otherwise declined and run on the SIMT kernel.
// Few tiles with a long K are split over K, with a finishing kernel that adds the partial
// tiles in a fixed order.
//
// Semantics: PrimDescriptor::{Contract, BatchedGemm}, tenferro-prims/src/lib.rs:156-168, 227-239.
#include <cuda.h>

#include "contract_common.cuh"
#include "contract_tables.h"
#include "ptx_sm100.cuh"

namespace tfb {

namespace {

constexpr int kBM = 128, kBK = 32;  // tile rows, k per stage (32 f32 = one 128-byte swizzle row)

// How one operand's tile maps onto its rank-5 tensor map.  A group (M, N or K) may hold up to
// two non-fusable modes (inner e1, outer e2); tiles either stay inside the inner mode (INNER:
// a tile is a range of the inner index for one outer index, padded with TMA's zero fill) or,
// when the inner extent divides the tile, pack several outer indices (PACK).
struct TcGeom {
    int mn_major;  // 0: K-major tile (K has unit stride), 1: MN-major tile (free group has unit stride)
    int pack;      // free group tiling: 0 INNER, 1 PACK
    int e1;        // extent of the free group's inner mode (of the whole group if it has one mode)
    int tiles1;    // INNER: tiles per inner-mode slice
};

struct TcArgs {
    char* c;
    const int64_t* c_b;
    const int64_t* c_m;
    const int64_t* c_n;
    // Column offsets in closed form when the N side of the output has at most two modes:
    // offset(n) = (n % cn_e1) * cn_s1 + (n / cn_e1) * cn_s2; cn_e1 == 0: use the c_n table.
    int cn_e1;
    int64_t cn_s1, cn_s2;
    int64_t dn_s1, dn_s2;  // the same two modes in the fused multiplier
    int64_t M, N, K, B;
    float alpha, beta;
    // Fused trailing multiplier D[b,m,n] (nullptr: none): C = alpha * (A B) . D + beta * C.
    const float* mul;
    const int64_t* d_b;
    const int64_t* d_m;
    const int64_t* d_n;
    TcGeom a, b;
    int k_e1, k_blocks1, num_kb;  // inner K extent, k-blocks per inner K slice, k-blocks in total
    int64_t tiles_m, tiles_n;
    int group_m;                  // m-tiles per raster group (L2 reuse)
    int k_split, kb_per_split;    // split-K: CTAs per output tile, k-blocks per CTA
    float* partial;               // split-K: [tile][split][BN cols][128 rows] raw sums
    int* status;
    // Output through TMA tensor stores (CTA-pair kernel): finished sums are staged in shared memory,
    // 32 rows x 32 columns per warp at a time, and leave as one bulk store each.  cm_e1: extent of
    // the output's unit-stride row mode (rows of one run); row r of the M group has tensor-map
    // coordinates (r % cm_e1, r / cm_e1), column n has (n % cn_e1, n / cn_e1).
    int c_tma;
    int cm_e1;
    // CTA-pair kernel: columns per half of a pair tile (a multiple of 32, at most 128).  A pair tile is
    // 2 * half_w columns wide and the MMAs have N = 2 * half_w, so an output with up to 256 columns
    // is ONE tile whose MMAs do no work on padding: half h holds columns [h * half_w, (h + 1) * half_w)
    // of the tile, in tensor memory as on the output side.
    int half_w;
};

// First row (linear index in the group), valid rows and tensor-map coordinates of free-group tile `t`.
struct TileRows {
    int64_t base;
    int valid, f1, f2;
};
__device__ __forceinline__ TileRows tile_rows(const TcGeom& g, int64_t t, int rows_per_tile, int64_t total) {
    // 32-bit divisions: tile numbers and row counts stay below 2^31 (checked on the host)
    TileRows r;
    const uint32_t t32 = (uint32_t)t;
    if (g.pack) {
        r.base = (int64_t)t32 * rows_per_tile;
        r.f1 = 0;
        r.f2 = (int)((uint32_t)r.base / (uint32_t)g.e1);
        r.valid = (int)min((int64_t)rows_per_tile, total - r.base);
    } else {
        const uint32_t f2 = t32 / (uint32_t)g.tiles1;
        r.f1 = (int)(t32 - f2 * (uint32_t)g.tiles1) * rows_per_tile;
        r.f2 = (int)f2;
        r.base = (int64_t)f2 * g.e1 + r.f1;
        r.valid = min(rows_per_tile, g.e1 - r.f1);
    }
    return r;
}

// Shared-memory matrix descriptor, sm_100 format: start address, leading and stride byte
// offsets in 16-byte units, version 1 at bit 46, layout type at bits 61-63
// (2: 128-byte swizzle of 16-byte units; 1: 128-byte swizzle of 32-byte units, the only
// layout the tensor core accepts for MN-major 32-bit operands).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46) | ((uint64_t)layout << 61);
}


// Raster of output tiles: m-tiles are visited in groups of `group_m` so that CTAs running
// together share B panels (and the A panels of the group) through L2.
struct TileCoord {
    int64_t batch, tm, tn;
};
__device__ __forceinline__ TileCoord decode_tile(int64_t tile, int64_t tiles_m, int64_t tiles_n, int group_m) {
    TileCoord t;
    const int64_t tiles_per_batch = tiles_m * tiles_n;
    t.batch = tile / tiles_per_batch;
    tile -= t.batch * tiles_per_batch;
    const int64_t group_sz = (int64_t)group_m * tiles_n;
    const int64_t grp = tile / group_sz;
    const int64_t first_m = grp * group_m;
    const int64_t rows_in_group = min((int64_t)group_m, tiles_m - first_m);
    const int64_t in_grp = tile - grp * group_sz;
    t.tm = first_m + in_grp % rows_in_group;
    t.tn = in_grp / rows_in_group;
    return t;
}

// a - trunc_tf32(a), exact in f32, plus half a TF32 ulp so that the tensor core's truncation of
// it rounds to nearest.  Integer operations only: conversion instructions run at a fraction
// of the ALU rate.
__device__ __forceinline__ float remainder_rounded(float a) {
    const float r = a - __uint_as_float(__float_as_uint(a) & 0xffffe000u);
    return __uint_as_float(__float_as_uint(r) + 0x1000u);
}

// a - trunc_tf32(a) without the rounding step: the exact remainder, to be rounded to bf16.
__device__ __forceinline__ float remainder_exact(float a) {
    return a - __uint_as_float(__float_as_uint(a) & 0xffffe000u);
}
// {lo, hi} as two bf16 in one register (lo in the lower half), round to nearest even.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// BF16C (the CTA-pair kernel): the two correction terms of 3xTF32 as ONE bf16 MMA of K = 16 per
// 8-deep k-step.  It adds remainder(a) b + a remainder(b) with all four rounded to bf16: the
// remainders are 2^-10 of the operands and bf16 rounds to 2^-9 relative, so the term is wrong by
// 2^-19 of the product at worst - the size of what 3xTF32 itself leaves out - for two MMAs' worth
// of tensor-pipe time (and power) per k-step instead of three.  A 16-deep bf16 k-step is 32 bytes
// per row, as an 8-deep TF32 one, so the correction tiles have the raw tiles' size.
//
// Which of the MMA's sixteen K slots holds what is free as long as both operands agree, and the
// order is chosen so that ONE 16-byte chunk of a raw K-major tile (four consecutive k of a row)
// becomes ONE 16-byte unit of the correction tile at the same place, in the raw tile's layout:
// slots 0-3 and 8-11 hold the first kind of value for k 0-3 and 4-7 of the k-step, slots 4-7 and
// 12-15 the second kind, the kinds being (remainder, value) in A and (value, remainder) in B.
// An MN-major tile ([32 k][32 mn] boxes, 32-byte units swizzled by k) becomes [64 k'][64 mn]
// blocks of 128-byte rows (16-byte units swizzled by k'): a thread takes the eight consecutive mn
// of one k (one 32-byte unit) and writes one unit into each of the two rows that are that k's slots.
__device__ __forceinline__ const char* mn_pair_src(const char* raw, uint32_t q) {
    // eight threads take the same k of two neighbouring boxes: the eight units of one new row
    const uint32_t box = ((q >> 8) << 1) | ((q >> 2) & 1u), k = (q >> 3) & 31u, a = q & 3u;
    return raw + (box << 12) + (k << 7) + (a << 5);
}
template <bool IS_B>
__device__ __forceinline__ void store_unit_kmajor(char* out, uint32_t c, const float4& v) {
    const uint32_t b0 = pack_bf16x2(v.x, v.y), b1 = pack_bf16x2(v.z, v.w);
    const uint32_t s0 = pack_bf16x2(remainder_exact(v.x), remainder_exact(v.y));
    const uint32_t s1 = pack_bf16x2(remainder_exact(v.z), remainder_exact(v.w));
    *reinterpret_cast<uint4*>(out + c * 16u) = IS_B ? make_uint4(b0, b1, s0, s1) : make_uint4(s0, s1, b0, b1);
}
// v0, v1: the eight consecutive mn of 32-byte unit q, in order
template <bool IS_B>
__device__ __forceinline__ void store_units_mnmajor(char* out, uint32_t q, const float4& v0, const float4& v1) {
    const uint32_t box = ((q >> 8) << 1) | ((q >> 2) & 1u), k = (q >> 3) & 31u, a = q & 3u;
    const uint4 big = make_uint4(pack_bf16x2(v0.x, v0.y), pack_bf16x2(v0.z, v0.w), pack_bf16x2(v1.x, v1.y), pack_bf16x2(v1.z, v1.w));
    const uint4 small = make_uint4(pack_bf16x2(remainder_exact(v0.x), remainder_exact(v0.y)),
                                   pack_bf16x2(remainder_exact(v0.z), remainder_exact(v0.w)),
                                   pack_bf16x2(remainder_exact(v1.x), remainder_exact(v1.y)),
                                   pack_bf16x2(remainder_exact(v1.z), remainder_exact(v1.w)));
    const uint32_t u = 4u * (box & 1u) + (a ^ (k & 3u));  // the 16-byte unit of these eight mn in the block's row
    // k's two slots among the sixteen of its k-step: (k & 3) + 8 (k / 4 & 1) and four further on
    const uint32_t row0 = ((k >> 3) << 4) + (k & 3u) + ((k & 4u) << 1);
    char* d0 = out + (box >> 1) * 8192u + row0 * 128u + (((u ^ row0) & 7u) << 4);
    char* d1 = out + (box >> 1) * 8192u + (row0 + 4u) * 128u + (((u ^ (row0 + 4u)) & 7u) << 4);
    *reinterpret_cast<uint4*>(d0) = IS_B ? big : small;
    *reinterpret_cast<uint4*>(d1) = IS_B ? small : big;
}
// One operand's four 16-byte loads of a round (K-major: four chunks; MN-major: two 32-byte units,
// read second half first by every other group of four threads so that a quarter-warp's loads
// cover all banks), and the matching stores.
template <bool MN, int NTHREADS>
__device__ __forceinline__ void load_round(const char* raw, int t, int r, uint32_t first, float4 (&v)[4]) {
    if constexpr (!MN) {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const float4*>(raw + (uint32_t)(t + (4 * r + i) * NTHREADS) * 16u);
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const char* src = mn_pair_src(raw, (uint32_t)(t + (2 * r + i) * NTHREADS));
            v[2 * i] = *reinterpret_cast<const float4*>(src + first);
            v[2 * i + 1] = *reinterpret_cast<const float4*>(src + (16u - first));
        }
    }
}
template <bool MN, bool IS_B, int NTHREADS>
__device__ __forceinline__ void store_round(char* out, int t, int r, uint32_t first, const float4 (&v)[4]) {
    if constexpr (!MN) {
#pragma unroll
        for (int i = 0; i < 4; ++i) store_unit_kmajor<IS_B>(out, (uint32_t)(t + (4 * r + i) * NTHREADS), v[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float4 lo = v[2 * i], hi = v[2 * i + 1];
            if (first) {
                const float4 tmp = lo;
                lo = hi;
                hi = tmp;
            }
            store_units_mnmajor<IS_B>(out, (uint32_t)(t + (2 * r + i) * NTHREADS), lo, hi);
        }
    }
}
// Both correction tiles (16 KB each, B behind A) of one stage by NTHREADS threads (t: this thread's
// number among them), in rounds of four chunks of each operand with the eight loads of a round
// issued first.
template <int NTHREADS, bool A_MN, bool B_MN>
__device__ __forceinline__ void convert_stage_bf16(const char* raw, char* out, int t) {
    constexpr int ROUNDS = 1024 / NTHREADS / 4;
    const uint32_t first = ((t >> 2) & 1) ? 16u : 0u;
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        float4 va[4], vb[4];
        load_round<A_MN, NTHREADS>(raw, t, r, first, va);
        load_round<B_MN, NTHREADS>(raw + 16384, t, r, first, vb);
        store_round<A_MN, false, NTHREADS>(out, t, r, first, va);
        store_round<B_MN, true, NTHREADS>(out + 16384, t, r, first, vb);
    }
}
template <int NTHREADS>
__device__ __forceinline__ void convert_stage_bf16(const char* raw, char* out, int t, bool a_mn, bool b_mn) {
    if (!a_mn && !b_mn) convert_stage_bf16<NTHREADS, false, false>(raw, out, t);
    else if (!a_mn) convert_stage_bf16<NTHREADS, false, true>(raw, out, t);
    else if (!b_mn) convert_stage_bf16<NTHREADS, true, false>(raw, out, t);
    else convert_stage_bf16<NTHREADS, true, true>(raw, out, t);
}

constexpr int kChunk = 8;           // k-blocks accumulated inside TMEM before promotion (K = 256)
constexpr int kSplitThreads = 256;  // warps 2..9

template <int BN>
struct TcCfg {
    static constexpr int A_BYTES = kBM * kBK * 4;  // 16 KB
    static constexpr int B_BYTES = BN * kBK * 4;
    static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);  // big + small of both operands
    static constexpr int STAGES = BN == 256 ? 2 : 3;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
    static constexpr int TMEM_COLS = 2 * BN;  // two f32 work accumulators, one column per n each
    static constexpr int COLS_PER_WARP = BN / 2;
    static_assert(kChunk >= STAGES, "promotion lag assumes a chunk spans at least the ring");
};

// The tensor core adds into its f32 accumulator with truncation, which shrinks a running
// sum by ~2^-26 per MMA: harmless for K of a few hundred, 4e-4 at K = 65536.  So TMEM only
// ever holds the sum of kChunk k-blocks (96 MMAs; the error then sits near 2e-6 relative Frobenius
// whatever K is - half of that with chunks of 4, at 5 % less speed); the split warps add each finished chunk
// to an f32 running sum in registers with ordinary round-to-nearest adds while the MMA
// thread fills the other work accumulator.
template <int BN>
__global__ void __launch_bounds__(64 + kSplitThreads, 1)
contract_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcArgs g) {
    using Cfg = TcCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int CPW = Cfg::COLS_PER_WARP;
    extern __shared__ char smem_raw[];
    // 128-byte swizzle atoms repeat every 1024 bytes: align the ring to that.
    char* smem = (char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t ring = smem_u32(smem);
    const uint32_t bars = ring + STAGES * Cfg::STAGE_BYTES;
    // barrier layout: full[s], split[s], empty[s], chunk_done[2], promoted[2], then the TMEM base word
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };
    auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
    auto bar_chunk = [&](int b) { return bars + 8u * (3 * STAGES + b); };
    auto bar_promoted = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
    const uint32_t tmem_word = bars + 8u * (3 * STAGES + 4);
    volatile uint32_t* tmem_word_ptr = (volatile uint32_t*)(smem + STAGES * Cfg::STAGE_BYTES + 8 * (3 * STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // split-K: consecutive CTAs take consecutive k ranges of one tile
    const int split = (int)(blockIdx.x % (unsigned)g.k_split);
    const int64_t tile_id = blockIdx.x / (unsigned)g.k_split;
    const TileCoord tc = decode_tile(tile_id, g.tiles_m, g.tiles_n, g.group_m);
    const int64_t bb = tc.batch, tm = tc.tm, tn = tc.tn;
    const TileRows tr_m = tile_rows(g.a, tm, kBM, g.M), tr_n = tile_rows(g.b, tn, BN, g.N);
    const int kb_first = split * g.kb_per_split;
    const int num_kb = min(g.kb_per_split, g.num_kb - kb_first);  // k-blocks of this CTA, numbered from 0 below
    const int num_chunks = (num_kb + kChunk - 1) / kChunk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_split(s), kSplitThreads / 32);
            mbar_init(bar_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_chunk(b), 1);
            mbar_init(bar_promoted(b), kSplitThreads / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_word, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_word_ptr;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t use = kb / STAGES;
                mbar_wait(bar_empty(s), (use & 1) ^ 1, g.status, 0x101);
                const uint32_t a_dst = ring + s * Cfg::STAGE_BYTES;
                const uint32_t b_dst = a_dst + Cfg::A_BYTES;
                mbar_expect_tx(bar_full(s), Cfg::A_BYTES + Cfg::B_BYTES);
                const int kg = kb_first + kb;
                const int k2 = kg / g.k_blocks1, k1 = (kg - k2 * g.k_blocks1) * kBK;
                if (g.a.mn_major) {
                    // [32 k][32 m] boxes, one per 32 rows of the tile; with packed tiling every
                    // box finds its own (inner, outer) coordinates from its linear row
                    for (int c = 0; c < kBM / 32; ++c) {
                        int f1 = tr_m.f1 + 32 * c, f2 = tr_m.f2;
                        if (g.a.pack) {
                            const int64_t row = tr_m.base + 32 * c;
                            f2 = (int)(row / g.a.e1);
                            f1 = (int)(row - (int64_t)f2 * g.a.e1);
                        }
                        tma_load_5d(a_dst + c * 4096, &map_a, bar_full(s), f1, f2, k1, k2, (int)bb);
                    }
                } else {
                    tma_load_5d(a_dst, &map_a, bar_full(s), k1, k2, tr_m.f1, tr_m.f2, (int)bb);
                }
                if (g.b.mn_major) {
                    for (int c = 0; c < BN / 32; ++c) {
                        int f1 = tr_n.f1 + 32 * c, f2 = tr_n.f2;
                        if (g.b.pack) {
                            const int64_t row = tr_n.base + 32 * c;
                            f2 = (int)(row / g.b.e1);
                            f1 = (int)(row - (int64_t)f2 * g.b.e1);
                        }
                        tma_load_5d(b_dst + c * 4096, &map_b, bar_full(s), f1, f2, k1, k2, (int)bb);
                    }
                } else {
                    // box rows are capped at 256 by the hardware; BN <= 256
                    tma_load_5d(b_dst, &map_b, bar_full(s), k1, k2, tr_n.f1, tr_n.f2, (int)bb);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)g.a.mn_major << 15) |
                                   ((uint32_t)g.b.mn_major << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
            // K-major: rows of 128 bytes, 8-row atoms 1024 bytes apart; a k step moves 32 bytes
            // inside the row.  MN-major: [32 k][32 mn] blocks 4096 bytes apart (leading offset),
            // swizzle atoms of 4 k-rows 512 bytes apart (stride offset); a k step of 8 moves 1024 bytes.
            const uint32_t a_lbo = g.a.mn_major ? 4096u : 16u, b_lbo = g.b.mn_major ? 4096u : 16u;
            const uint32_t a_sbo = g.a.mn_major ? 512u : 1024u, b_sbo = g.b.mn_major ? 512u : 1024u;
            const uint32_t a_lay = g.a.mn_major ? 1u : 2u, b_lay = g.b.mn_major ? 1u : 2u;
            const uint32_t a_step = g.a.mn_major ? 1024u : 32u, b_step = g.b.mn_major ? 1024u : 32u;
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t use = kb / STAGES;
                const int chunk = kb / kChunk, buf = chunk & 1;
                const bool chunk_first = kb % kChunk == 0;
                const bool chunk_last = (kb % kChunk == kChunk - 1) || kb == num_kb - 1;
                if (chunk_first && chunk >= 2) {
                    // the work accumulator is free once the chunk it held has been promoted
                    mbar_wait(bar_promoted(buf), ((uint32_t)(chunk >> 1) - 1) & 1, g.status, 0x105);
                    tc_fence_after();
                }
                mbar_wait(bar_split(s), use & 1, g.status, 0x102);
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                const uint32_t a_big = ring + s * Cfg::STAGE_BYTES;
                const uint32_t b_big = a_big + Cfg::A_BYTES;
                const uint32_t a_small = b_big + Cfg::B_BYTES;
                const uint32_t b_small = a_small + Cfg::A_BYTES;
#pragma unroll
                for (int ks = 0; ks < kBK / 8; ++ks) {
                    const uint64_t da_big = smem_desc(a_big + ks * a_step, a_lbo, a_sbo, a_lay);
                    const uint64_t da_small = smem_desc(a_small + ks * a_step, a_lbo, a_sbo, a_lay);
                    const uint64_t db_big = smem_desc(b_big + ks * b_step, b_lbo, b_sbo, b_lay);
                    const uint64_t db_small = smem_desc(b_small + ks * b_step, b_lbo, b_sbo, b_lay);
                    tc_mma_tf32(tmem_d, da_small, db_big, idesc, !(chunk_first && ks == 0));
                    tc_mma_tf32(tmem_d, da_big, db_small, idesc, 1);
                    tc_mma_tf32(tmem_d, da_big, db_big, idesc, 1);
                }
                tc_commit(bar_empty(s));                  // stage reusable once these MMAs have read it
                if (chunk_last) tc_commit(bar_chunk(buf));  // work accumulator complete
            }
        }
    } else {
        // ---------------------------------------------------------------- split + promote, then epilogue
        const int t = threadIdx.x - 64;  // 0..255
        // warp w may touch TMEM lanes 32 * (w % 4) .. + 31; lane = row of the tile.  Warps 2-5
        // own the first half of the columns, warps 6-9 the second.
        const int lane_grp = warp & 3;
        const int col0 = ((warp - 2) >> 2) * CPW;
        const uint32_t tmem_mine = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)col0;
        float acc[CPW];
#pragma unroll
        for (int j = 0; j < CPW; ++j) acc[j] = 0.f;
        int next_promote = 0;
        auto promote = [&](int chunk) {
            const int buf = chunk & 1;
            // one lane polls, the warp follows: mbarrier operations of 32 lanes on one word serialise
            if (lane == 0) mbar_wait(bar_chunk(buf), (uint32_t)(chunk >> 1) & 1, g.status, 0x104);
            __syncwarp();
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < CPW; c0 += 32) {
                uint32_t r[32];
                tc_ld32(tmem_mine + (uint32_t)(buf * BN + c0), r);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(r[j]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_promoted(buf));
        };
        for (int kb = 0; kb < num_kb; ++kb) {
            const int s = kb % STAGES;
            const uint32_t use = kb / STAGES;
            if (lane == 0) mbar_wait(bar_full(s), use & 1, g.status, 0x103);
            __syncwarp();
            char* big = smem + (size_t)s * Cfg::STAGE_BYTES;
            char* small = big + Cfg::A_BYTES + Cfg::B_BYTES;
            constexpr int CHUNKS = (Cfg::A_BYTES + Cfg::B_BYTES) / 16;
#pragma unroll 4
            for (int c = t; c < CHUNKS; c += kSplitThreads) {
                const float4 v = *reinterpret_cast<const float4*>(big + (size_t)c * 16);
                float4 sm;
                // the tensor core reads only the upper 19 bits of each f32: the raw tile already is
                // the truncated "big" operand; the remainder is exact in f32 and rounded to tf32
                sm.x = remainder_rounded(v.x);
                sm.y = remainder_rounded(v.y);
                sm.z = remainder_rounded(v.z);
                sm.w = remainder_rounded(v.w);
                *reinterpret_cast<float4*>(small + (size_t)c * 16) = sm;
            }
            fence_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_split(s));
            // A chunk whose last k-block lies STAGES behind has certainly retired: the stage
            // just split could only be loaded after that k-block's MMAs freed it.
            while (next_promote < num_chunks &&
                   min((next_promote + 1) * kChunk, num_kb) - 1 + STAGES <= kb)
                promote(next_promote++);
        }
        while (next_promote < num_chunks) promote(next_promote++);

        const int row = lane_grp * 32 + lane;
        if (g.k_split > 1) {
            // raw partial sums, rows fastest; the finishing kernel adds the splits in order
            float* P = g.partial + ((size_t)(tile_id * g.k_split + split) * BN + col0) * kBM + row;
#pragma unroll
            for (int j = 0; j < CPW; ++j) P[(size_t)j * kBM] = acc[j];
        } else if (row < tr_m.valid) {
            float* C = reinterpret_cast<float*>(g.c) + g.c_b[bb];
            const int64_t cm = g.c_m[tr_m.base + row];
            const bool read_c = g.beta != 0.f;
            if (g.mul) {
                // multiplier values first, all loads in flight together (see store_acc_slice)
                const float* D = g.mul + g.d_b[bb] + g.d_m[tr_m.base + row];
#pragma unroll
                for (int j = 0; j < CPW; ++j)
                    if (col0 + j < tr_n.valid) acc[j] *= D[g.d_n[tr_n.base + col0 + j]];
            }
#pragma unroll
            for (int j = 0; j < CPW; ++j) {
                const int col = col0 + j;
                if (col < tr_n.valid) {
                    float* p = C + cm + g.c_n[tr_n.base + col];
                    float v = g.alpha * acc[j];
                    if (read_c) v += g.beta * *p;
                    *p = v;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// Split-K finish: C tile = alpha * (sum of the splits' partial tiles, in split order) + beta * C.
constexpr int kFinishCols = 8;  // columns of a tile per finishing CTA
template <int BN>
__global__ void __launch_bounds__(256) tf32x3_splitk_finish_kernel(TcArgs g) {
    const int64_t tile_id = blockIdx.x;
    const TileCoord tc = decode_tile(tile_id, g.tiles_m, g.tiles_n, g.group_m);
    const int64_t bb = tc.batch, tm = tc.tm, tn = tc.tn;
    const TileRows tr_m = tile_rows(g.a, tm, kBM, g.M), tr_n = tile_rows(g.b, tn, BN, g.N);
    const int row = threadIdx.x & (kBM - 1);
    if (row >= tr_m.valid) return;
    float* C = reinterpret_cast<float*>(g.c) + g.c_b[bb];
    const int64_t cm = g.c_m[tr_m.base + row];
    const bool read_c = g.beta != 0.f;
    const float* P = g.partial + (size_t)tile_id * g.k_split * BN * kBM + row;
    const float* D = g.mul ? g.mul + g.d_b[bb] + g.d_m[tr_m.base + row] : nullptr;
    // blockIdx.y takes kFinishCols columns of the tile; two columns are in flight per pass
    const int col_end = min(tr_n.valid, (int)(blockIdx.y + 1) * kFinishCols);
    for (int col = blockIdx.y * kFinishCols + threadIdx.x / kBM; col < col_end; col += 256 / kBM) {
        float sum = 0.f;
#pragma unroll 8
        for (int s = 0; s < g.k_split; ++s) sum += P[((size_t)s * BN + col) * kBM];
        float* p = C + cm + g.c_n[tr_n.base + col];
        float v = g.alpha * sum;
        if (D) v *= D[g.d_n[tr_n.base + col]];
        if (read_c) v += g.beta * *p;
        *p = v;
    }
}

// ------------------------------------------------------------------ CTA-pair variant
// Two CTAs of a cluster share one 256 x 256 tile of C through tcgen05.mma.cta_group::2: each
// CTA stages its own 128 rows of A and only HALF of the B tile (128 of the 256 columns), the
// pair's tensor cores exchange the B halves, and each CTA ends up with its 128 x 256 part of
// the product in its own tensor memory.  Per k-block a CTA moves a third less through shared
// memory than the single-CTA kernel (which is bound by exactly that), in 64 KB stages instead
// of 96 KB, so three stages fit.
//
// Roles per CTA are those of the single-CTA kernel, except that only the leader (rank 0)
// issues MMAs.  Barriers:
//   full[s]      own CTA   TMA bytes of stage s landed                     -> own converters
//   split[s]     LEADER    both CTAs' converters are done with stage s     -> MMA thread
//   empty[s]     each CTA  MMAs that read stage s retired (commit to both) -> own producer
//   chunk[b]     each CTA  work accumulator b complete (commit to both)    -> own converters
//   promoted[b]  LEADER    both CTAs have read work accumulator b          -> MMA thread
// Arrivals on the leader's barriers from the other CTA go to the mapped address with CTA-scope
// release semantics (see mbar_arrive_cluster); commits go to each CTA's barrier by an
// instruction of its own, so every instruction here addresses exactly one CTA.
// Output boxes of the TMA-store epilogue: 32 rows (one warp's TMEM lanes) x kBoxCols columns.
constexpr int kBoxCols = 32;
constexpr int kBoxBytes = 32 * kBoxCols * 4;

struct PairCfg {
    static constexpr int BN = 256;                  // tile columns of the pair
    static constexpr int A_BYTES = kBM * kBK * 4;   // 16 KB: this CTA's 128 rows
    static constexpr int B_BYTES = 128 * kBK * 4;   // 16 KB: this CTA's 128 of the 256 columns
    static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);
    static constexpr int STAGES = 3;
    static constexpr int BAR_BYTES = 256;
    // staging of output boxes for TMA stores: 8 warps x one 4 KB box (general kernel) or 4 drain
    // warps x two boxes (short-K kernel)
    static constexpr int OUT_STAGE_BYTES = 8 * kBoxBytes;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + OUT_STAGE_BYTES + 1024;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr int COLS_PER_WARP = BN / 2;
    static_assert(kChunk >= STAGES, "promotion lag assumes a chunk spans at least the ring");
    static_assert((STAGES * STAGE_BYTES + BAR_BYTES) % 128 == 0, "the output staging area must be 128-byte aligned");
};

// Finished columns [kBoxCols Q, kBoxCols (Q + 1)) of one thread's row, scaled, into the warp's
// staging box (column-major: 32 rows of one column are 128 contiguous bytes, so the warp's stores
// to shared memory are conflict-free and the box is what a {32, kBoxCols} TMA store expects).
template <int Q, int N>
__device__ __forceinline__ void stage_acc_cols(const float (&acc)[N], float* box_lane, float alpha) {
#pragma unroll
    for (int jj = 0; jj < kBoxCols; ++jj) box_lane[jj * 32] = alpha * acc[kBoxCols * Q + jj];
}

// Columns [Q, Q + 1) * ceil(N / SLICES) of one thread's row of finished sums.  Column offsets
// follow the (at most two) output modes of the N side in closed form - no table loads in the
// way; indices into `acc` are compile-time so the sums stay in registers.
template <int Q, int SLICES, int N, bool MUL>
__device__ __forceinline__ void store_acc_slice(const float (&acc)[N], float* row, int col0, int e1, int64_t s1, int64_t s2,
                                                int valid, float alpha, float beta, const float* drow, int64_t ds1,
                                                int64_t ds2) {
    constexpr int W = (N + SLICES - 1) / SLICES;
    constexpr int j0 = Q * W;
    if (j0 >= valid) return;
    const bool read_c = beta != 0.f;
    const int n0 = col0 + j0, outer = n0 / e1;
    int inner = n0 - outer * e1;
    float* p = row + inner * s1 + outer * s2;
    const int64_t wrap = s2 - (int64_t)e1 * s1;
    // The fused multiplier's row walks the same two modes with its own strides.  Its values are
    // all fetched before the first store: a load issued after a store through an unrelated
    // pointer would wait for it, and the slice would pay one memory round trip per column.
    float dv[MUL ? W : 1];
    if constexpr (MUL) {
        int64_t d = inner * ds1 + outer * ds2;
        const int64_t dwrap = ds2 - (int64_t)e1 * ds1;
        int din = inner;
#pragma unroll
        for (int jj = 0; jj < W; ++jj) {
            dv[jj] = (j0 + jj < N && j0 + jj < valid) ? drow[d] : 1.f;
            d += ds1;
            if (++din == e1) {
                din = 0;
                d += dwrap;
            }
        }
    }
#pragma unroll
    for (int jj = 0; jj < W; ++jj) {
        if (j0 + jj < N && j0 + jj < valid) {
            float v = alpha * acc[j0 + jj < N ? j0 + jj : 0];
            if constexpr (MUL) v *= dv[jj];
            if (read_c) v += beta * *p;
            *p = v;
        }
        p += s1;
        if (++inner == e1) {
            inner = 0;
            p += wrap;
        }
    }
}

// One unit of work of a CTA pair: a 256 x 256 pair tile (128-row m-tiles 2 tmp, 2 tmp + 1, one per
// CTA, x 128-column n-tiles 2 tnp, 2 tnp + 1) and, with split-K, one k range of it.
struct PairWork {
    int64_t batch, pair_tile;
    int split, kb_first, num_kb;
    TileRows tr_m;      // this CTA's rows
    TileRows tr_n[2];   // the two column halves of the tile
};
// decode_tile in 32-bit arithmetic (the host keeps the number of work items below 2^31): a 64-bit
// division costs several times a 32-bit one, and these run in the threads whose latency the
// pipeline feels.
__device__ __forceinline__ TileCoord decode_tile32(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_m) {
    TileCoord t;
    const uint32_t tiles_per_batch = tiles_m * tiles_n;
    const uint32_t batch = tile / tiles_per_batch;
    tile -= batch * tiles_per_batch;
    const uint32_t group_sz = group_m * tiles_n;
    const uint32_t grp = tile / group_sz;
    const uint32_t first_m = grp * group_m;
    const uint32_t rows_in_group = min(group_m, tiles_m - first_m);
    const uint32_t in_grp = tile - grp * group_sz;
    const uint32_t tn = in_grp / rows_in_group;
    t.batch = batch;
    t.tm = first_m + (in_grp - tn * rows_in_group);
    t.tn = tn;
    return t;
}
__device__ __forceinline__ PairWork pair_work(const TcArgs& g, int64_t w, uint32_t rank) {
    PairWork pw;
    const int64_t tiles_mp = (g.tiles_m + 1) / 2, tiles_np = (g.tiles_n + 1) / 2;
    const uint32_t w32 = (uint32_t)w, ks = (uint32_t)g.k_split;
    const uint32_t pt = w32 / ks;
    pw.split = (int)(w32 - pt * ks);
    pw.pair_tile = pt;
    const TileCoord tc = decode_tile32(pt, (uint32_t)tiles_mp, (uint32_t)tiles_np, (uint32_t)g.group_m);
    pw.batch = tc.batch;
    // A tile past the end (odd tile counts) has coordinates outside the tensor: TMA fills it
    // with zeros and nothing of it is stored.
    pw.tr_m = tile_rows(g.a, 2 * tc.tm + rank, kBM, g.M);
    if (2 * tc.tm + rank >= g.tiles_m) pw.tr_m.valid = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        pw.tr_n[h] = tile_rows(g.b, 2 * tc.tn + h, g.half_w, g.N);
        if (2 * tc.tn + h >= g.tiles_n) pw.tr_n[h].valid = 0;
    }
    pw.kb_first = pw.split * g.kb_per_split;
    pw.num_kb = min(g.kb_per_split, g.num_kb - pw.kb_first);
    return pw;
}

// The k-blocks of work item w alone (what pair_work reports as num_kb), without the tile decode and
// its 64-bit divisions: all that the MMA thread and the converting warps need to know.
__device__ __forceinline__ int pair_num_kb(const TcArgs& g, int64_t w) {
    const int split = (int)(w % g.k_split);
    return min(g.kb_per_split, g.num_kb - split * g.kb_per_split);
}

// Threads of the pair kernel: the lead warps (producer, MMA issuer and, in the long-K variant, two
// warps that only hand their registers over) and eight worker warps.
constexpr int pair_lead_threads(bool shortk) { return shortk ? 64 : 128; }
constexpr int pair_threads(bool shortk) { return pair_lead_threads(shortk) + kSplitThreads; }
// Registers.  The short-K variant runs ten warps in the 168 registers per thread that three warps
// to a scheduler partition of 16 K registers leave.  The long-K variant's workers hold a 128-wide
// row of running sums each and want more: it runs TWELVE warps at 168, the first warpgroup gives
// its registers up to kLeadRegs per thread and the two worker warpgroups take kWorkerRegs (a
// partition then holds kLeadRegs + 2 kWorkerRegs of its 512 per lane).
constexpr int kLeadRegs = 72, kWorkerRegs = 216;
static_assert(kLeadRegs + 2 * kWorkerRegs <= 512 && pair_threads(false) * 168 >= 128 * kLeadRegs + 256 * kWorkerRegs,
              "the registers the workers take are the ones the lead warps gave up");

// MUL: the launch carries a fused multiplier (g.mul != nullptr).  A separate instantiation keeps the
// multiplier's registers out of the plain kernel.
// SHORTK: every work item fits one TMEM accumulation chunk (K <= kChunk k-blocks, no split-K), so
// the sums in tensor memory are final.  Half of the converter warps then only convert; the other
// half only drain finished accumulators to the output (tcgen05.ld -> global stores).  Stores that
// wait for the memory system no longer hold up the conversion the tensor cores are waiting for:
// a short-K product writes its output at DRAM speed WHILE the next tiles are multiplied.
// BF16C: the two correction terms of a k-step as one bf16 MMA on correction tiles (see
// convert_stage_bf16) instead of two TF32 MMAs on remainder tiles.
template <bool MUL, bool SHORTK, bool BF16C>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_threads(SHORTK), 1)
contract_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            const __grid_constant__ CUtensorMap map_c, TcArgs g) {
    using Cfg = PairCfg;
    constexpr int STAGES = Cfg::STAGES, BN = Cfg::BN, CPW = Cfg::COLS_PER_WARP;
    extern __shared__ char smem_raw[];
    // Both CTAs must lay their rings out identically: descriptors and barrier offsets are
    // interpreted in each CTA's own shared memory.  The dynamic segment starts at the same
    // offset in every CTA of a launch, so the same rounding gives the same layout.
    char* smem = (char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t ring = smem_u32(smem);
    const uint32_t bars = ring + STAGES * Cfg::STAGE_BYTES;
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_split = [&](int s) { return bars + 8u * (STAGES + s); };
    auto bar_empty = [&](int s) { return bars + 8u * (2 * STAGES + s); };
    auto bar_chunk = [&](int b) { return bars + 8u * (3 * STAGES + b); };
    auto bar_promoted = [&](int b) { return bars + 8u * (3 * STAGES + 2 + b); };
    const uint32_t tmem_word = bars + 8u * (3 * STAGES + 4);
    volatile uint32_t* tmem_word_ptr = (volatile uint32_t*)(smem + STAGES * Cfg::STAGE_BYTES + 8 * (3 * STAGES + 4));
    // staging area of the TMA-store epilogue (see PairCfg::OUT_STAGE_BYTES)
    const uint32_t out_stage = bars + Cfg::BAR_BYTES;
    float* out_stage_ptr = (float*)(smem + STAGES * Cfg::STAGE_BYTES + Cfg::BAR_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    constexpr int kWarps = kSplitThreads / 32;
    constexpr int kLead = pair_lead_threads(SHORTK), kLeadWarps = kLead / 32;  // threads and warps before the workers
    // warps per CTA that arrive on the "converted" and on the "accumulator drained" barriers
    constexpr int kRoleWarps = SHORTK ? kWarps / 2 : kWarps;

    // Persistent: this pair takes work items w0, w0 + wstep, ...  Every role walks the same
    // sequence with running counters (k-blocks for the stage ring, chunks for the two work
    // accumulators), so the producer is already loading the next tile while the converter
    // warps store the current one, and barriers, tensor memory and the cluster handshake are
    // set up once per CTA instead of once per tile.
    const int64_t n_work = ((g.tiles_m + 1) / 2) * ((g.tiles_n + 1) / 2) * g.B * g.k_split;
    const int64_t w0 = blockIdx.x >> 1, wstep = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_split(s), 2 * kRoleWarps);
            mbar_init(bar_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_chunk(b), 1);
            mbar_init(bar_promoted(b), 2 * kRoleWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_word, Cfg::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();  // barriers of both CTAs exist before anyone arrives on the peer's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_word_ptr;

    if (warp < kLeadWarps) {
    if constexpr (!SHORTK) reg_release<kLeadRegs>();
    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (each CTA its own tiles)
        if (lane == 0) {
            uint32_t it = 0;
            int p_stage = 0;
            uint32_t p_parity = 0;
            PairWork pw_next = pair_work(g, w0, rank);
            for (int64_t w = w0; w < n_work; w += wstep) {
            const PairWork pw = pw_next;
            const TileRows tr_m = pw.tr_m, tr_nl = rank ? pw.tr_n[1] : pw.tr_n[0];  // tr_nl: the half of B this CTA stages
            const int64_t bb = pw.batch;
            // Coordinates of the four 32-row boxes of an MN-major tile, once per work item: with packed
            // tiling every box finds its own (inner, outer) pair from its linear row, and a division
            // per box and k-block in this thread delays every load of the tile (an i-slice with 64 rows
            // per run: 86 ms instead of 72 ms for M = 8192, N = 16384, K = 65536).
            int a_f1[kBM / 32], a_f2[kBM / 32], b_f1[4], b_f2[4];
#pragma unroll
            for (int c = 0; c < kBM / 32; ++c) {
                a_f1[c] = tr_m.f1 + 32 * c;
                a_f2[c] = tr_m.f2;
                if (g.a.pack) {
                    const int64_t row = tr_m.base + 32 * c;
                    a_f2[c] = (int)(row / g.a.e1);
                    a_f1[c] = (int)(row - (int64_t)a_f2[c] * g.a.e1);
                }
                b_f1[c] = tr_nl.f1 + 32 * c;
                b_f2[c] = tr_nl.f2;
                if (g.b.pack) {
                    const int64_t row = tr_nl.base + 32 * c;
                    b_f2[c] = (int)(row / g.b.e1);
                    b_f1[c] = (int)(row - (int64_t)b_f2[c] * g.b.e1);
                }
            }
            // k coordinates advance without a division per k-block (this thread's latency is the loads')
            int k2 = pw.kb_first / g.k_blocks1, k1b = pw.kb_first - k2 * g.k_blocks1;
            for (int kb = 0; kb < pw.num_kb; ++kb, ++it) {
                // stage number and pass parity are counted, not divided out: whatever this thread
                // does between the stage becoming free and the loads going out delays the tile
                const int s = p_stage;
                const int k1 = k1b * kBK;
                const uint32_t a_dst = ring + s * Cfg::STAGE_BYTES;
                const uint32_t b_dst = a_dst + Cfg::A_BYTES;
                mbar_wait(bar_empty(s), p_parity ^ 1, g.status, 0x111);
                if (++p_stage == STAGES) {
                    p_stage = 0;
                    p_parity ^= 1;
                }
                mbar_expect_tx(bar_full(s), Cfg::A_BYTES + Cfg::B_BYTES);
                if (g.a.mn_major) {
#pragma unroll
                    for (int c = 0; c < kBM / 32; ++c)
                        tma_load_5d(a_dst + c * 4096, &map_a, bar_full(s), a_f1[c], a_f2[c], k1, k2, (int)bb);
                } else {
                    tma_load_5d(a_dst, &map_a, bar_full(s), k1, k2, tr_m.f1, tr_m.f2, (int)bb);
                }
                if (g.b.mn_major) {
#pragma unroll
                    for (int c = 0; c < 128 / 32; ++c)
                        tma_load_5d(b_dst + c * 4096, &map_b, bar_full(s), b_f1[c], b_f2[c], k1, k2, (int)bb);
                } else {
                    tma_load_5d(b_dst, &map_b, bar_full(s), k1, k2, tr_nl.f1, tr_nl.f2, (int)bb);
                }
                if (++k1b == g.k_blocks1) {
                    k1b = 0;
                    ++k2;
                }
                // the next work item is decoded behind this one's first loads, not in front of its own
                if (kb == 0 && w + wstep < n_work) pw_next = pair_work(g, w + wstep, rank);
            }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)g.a.mn_major << 15) |
                                   ((uint32_t)g.b.mn_major << 16) | ((uint32_t)((2 * g.half_w) >> 3) << 17) |
                                   ((uint32_t)((2 * kBM) >> 4) << 24);
            const uint32_t a_lbo = g.a.mn_major ? 4096u : 16u, b_lbo = g.b.mn_major ? 4096u : 16u;
            const uint32_t a_sbo = g.a.mn_major ? 512u : 1024u, b_sbo = g.b.mn_major ? 512u : 1024u;
            const uint32_t a_lay = g.a.mn_major ? 1u : 2u, b_lay = g.b.mn_major ? 1u : 2u;
            const uint32_t a_step = g.a.mn_major ? 1024u : 32u, b_step = g.b.mn_major ? 1024u : 32u;
            uint32_t it = 0, ch0 = 0;  // k-blocks and chunks issued before this work item
            // Descriptors of stage 0, k-step 0; those of stage s and k-step ks differ only in the start
            // address field (bits 0-13, in 16-byte units), so they follow by one addition each.  What
            // this thread computes between a stage being converted and its first MMA delays the tile.
            const uint64_t da_big0 = smem_desc(ring, a_lbo, a_sbo, a_lay);
            const uint64_t db_big0 = smem_desc(ring + Cfg::A_BYTES, b_lbo, b_sbo, b_lay);
            // The second operands: TF32 remainders in the raw tiles' layout, or (BF16C) bf16 correction
            // tiles - K-major ones in the same layout, MN-major ones as [64 k'][64 mn] blocks 8192
            // bytes apart with 8-row swizzle atoms 1024 bytes apart, a 16-deep k-step moving 2048 bytes.
            const uint32_t a2_lbo = BF16C && g.a.mn_major ? 8192u : a_lbo, b2_lbo = BF16C && g.b.mn_major ? 8192u : b_lbo;
            const uint32_t a2_sbo = BF16C ? 1024u : a_sbo, b2_sbo = BF16C ? 1024u : b_sbo;
            const uint32_t a2_lay = BF16C ? 2u : a_lay, b2_lay = BF16C ? 2u : b_lay;
            const uint32_t a2_step = BF16C && g.a.mn_major ? 2048u : a_step, b2_step = BF16C && g.b.mn_major ? 2048u : b_step;
            const uint64_t da_small0 = smem_desc(ring + Cfg::A_BYTES + Cfg::B_BYTES, a2_lbo, a2_sbo, a2_lay);
            const uint64_t db_small0 = smem_desc(ring + 2 * Cfg::A_BYTES + Cfg::B_BYTES, b2_lbo, b2_sbo, b2_lay);
            const uint32_t a_inc = a_step >> 4, b_inc = b_step >> 4, a2_inc = a2_step >> 4, b2_inc = b2_step >> 4;
            // bf16 x bf16 -> f32, same shape and majors
            const uint32_t idesc_c = (idesc & ~((7u << 7) | (7u << 10))) | (1u << 7) | (1u << 10);
            int m_stage = 0;
            uint32_t m_parity = 0;
            for (int64_t w = w0; w < n_work; w += wstep) {
            const int num_kb = pair_num_kb(g, w);
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const int s = m_stage;
                const uint32_t chunk = ch0 + kb / kChunk;
                const int buf = chunk & 1;
                const bool chunk_first = kb % kChunk == 0;
                const bool chunk_last = (kb % kChunk == kChunk - 1) || kb == num_kb - 1;
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                const uint32_t stage_off = (uint32_t)(s * (Cfg::STAGE_BYTES >> 4));
                uint64_t da_big = da_big0 + stage_off, da_small = da_small0 + stage_off;
                uint64_t db_big = db_big0 + stage_off, db_small = db_small0 + stage_off;
                if (chunk_first && chunk >= 2) {
                    mbar_wait_cluster(bar_promoted(buf), ((uint32_t)(chunk >> 1) - 1) & 1, g.status, 0x115);
                    tc_fence_after();
                }
                mbar_wait_cluster(bar_split(s), m_parity, g.status, 0x112);
                tc_fence_after();
                if (++m_stage == STAGES) {
                    m_stage = 0;
                    m_parity ^= 1;
                }
#pragma unroll
                for (int ks = 0; ks < kBK / 8; ++ks) {
                    if constexpr (BF16C) {
                        tc_mma_f16_pair(tmem_d, da_small, db_small, idesc_c, !(chunk_first && ks == 0));
                    } else {
                        tc_mma_tf32_pair(tmem_d, da_small, db_big, idesc, !(chunk_first && ks == 0));
                        tc_mma_tf32_pair(tmem_d, da_big, db_small, idesc, 1);
                    }
                    tc_mma_tf32_pair(tmem_d, da_big, db_big, idesc, 1);
                    da_big += a_inc;
                    da_small += a2_inc;
                    db_big += b_inc;
                    db_small += b2_inc;
                }
                tc_commit_pair(bar_empty(s));
                tc_commit_pair(map_to_cta(bar_empty(s), 1));
                if (chunk_last) {
                    tc_commit_pair(bar_chunk(buf));
                    tc_commit_pair(map_to_cta(bar_chunk(buf), 1));
                }
            }
            ch0 += (uint32_t)((num_kb + kChunk - 1) / kChunk);
            }
        }
    }
    } else if constexpr (SHORTK) {
        const uint32_t leader_split0 = map_to_cta(bar_split(0), 0), leader_promoted0 = map_to_cta(bar_promoted(0), 0);
        if (warp < kLeadWarps + kRoleWarps) {
            // ------------------------------------------------------------ converters only (warps 2-5)
            constexpr int kConvThreads = kRoleWarps * 32;
            const int t = threadIdx.x - kLead;
            uint32_t it = 0;
            for (int64_t w = w0; w < n_work; w += wstep) {
                const int num_kb = pair_num_kb(g, w);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t use = it / STAGES;
                    if (lane == 0) mbar_wait(bar_full(s), use & 1, g.status, 0x113);
                    __syncwarp();
                    char* big = smem + (size_t)s * Cfg::STAGE_BYTES;
                    char* small = big + Cfg::A_BYTES + Cfg::B_BYTES;
                    constexpr int CHUNKS = (Cfg::A_BYTES + Cfg::B_BYTES) / 16;
                    if constexpr (BF16C) {
                        static_assert(Cfg::A_BYTES == 16384 && Cfg::B_BYTES == 16384, "convert_stage_bf16 is written for 16 KB tiles");
                        convert_stage_bf16<kConvThreads>(big, small, t, g.a.mn_major != 0, g.b.mn_major != 0);
                    } else {
#pragma unroll 4
                        for (int c = t; c < CHUNKS; c += kConvThreads) {
                            const float4 v = *reinterpret_cast<const float4*>(big + (size_t)c * 16);
                            float4 sm;
                            sm.x = remainder_rounded(v.x);
                            sm.y = remainder_rounded(v.y);
                            sm.z = remainder_rounded(v.z);
                            sm.w = remainder_rounded(v.w);
                            *reinterpret_cast<float4*>(small + (size_t)c * 16) = sm;
                        }
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(leader_split0 + 8u * s);
                }
            }
        } else {
            // ------------------------------------------------------------ drain warps (6-9): TMEM -> C
            // One chunk per work item, so work item number = chunk number; the two accumulators
            // alternate and the MMA thread reuses one only after all drain warps released it.
            const int lane_grp = warp & 3;
            const int row = lane_grp * 32 + lane;
            const uint32_t tmem_row = tmem_base + ((uint32_t)(lane_grp * 32) << 16);
            const bool read_c = g.beta != 0.f;
            // TMA-store path: two 2 KB boxes per drain warp, used alternately
            const int slot0 = (warp - kLeadWarps - kRoleWarps) * 2;
            uint32_t n_boxes = 0;
            uint32_t chunk = 0;
            for (int64_t w = w0; w < n_work; w += wstep, ++chunk) {
                const PairWork pw = pair_work(g, w, rank);
                const int buf = chunk & 1;
                if (lane == 0) mbar_wait(bar_chunk(buf), (chunk >> 1) & 1, g.status, 0x116);
                __syncwarp();
                tc_fence_after();
                const bool live = row < pw.tr_m.valid;
                if (!MUL && g.c_tma) {
                    static_assert(kBoxCols == 32, "boxes are read from tensor memory with one 32-column load");
                    // 32 rows x 32 columns at a time: tcgen05.ld -> registers -> shared memory -> one bulk
                    // tensor store.  The warp's global stores no longer sit in the load/store queue that
                    // the converter warps' shared-memory traffic goes through, and the read of the next
                    // box is in flight while this one is staged.
                    const bool rows_live = 32 * lane_grp < pw.tr_m.valid;  // warp-uniform
                    const int row_lin = (int)pw.tr_m.base + 32 * lane_grp;
                    const int m_in = row_lin % g.cm_e1, m_out = row_lin / g.cm_e1;
                    // box b of the tile: half b / 4, columns 32 (b % 4) .. + 31 of it
                    auto box_valid = [&](int b) { return rows_live && pw.tr_n[b >> 2].valid > (b & 3) * 32; };
                    auto box_taddr = [&](int b) { return tmem_row + (uint32_t)(buf * BN + (b >> 2) * g.half_w + (b & 3) * 32); };
                    uint32_t r[2][32];
                    bool in_flight = false;  // the read of box b was issued while box b - 1 was staged
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        if (!box_valid(b)) {
                            in_flight = false;
                            continue;
                        }
                        if (!in_flight) tc_ld32(box_taddr(b), r[b & 1]);
                        tc_wait_ld();
                        in_flight = b + 1 < 8 && box_valid(b + 1);
                        if (in_flight) tc_ld32(box_taddr(b + 1), r[(b + 1) & 1]);
                        const int slot = slot0 + (int)(n_boxes & 1u);
                        if (lane == 0) bulk_wait_read<1>();  // the box written two stores ago has been read
                        __syncwarp();
                        float* box = out_stage_ptr + slot * (kBoxBytes / 4) + lane;
#pragma unroll
                        for (int j = 0; j < 32; ++j) box[j * 32] = g.alpha * __uint_as_float(r[b & 1][j]);
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const TileRows trn = pw.tr_n[b >> 2];
                            const int col = (int)trn.base + (b & 3) * 32;
                            tma_store_5d(&map_c, out_stage + (uint32_t)(slot * kBoxBytes), m_in, m_out, col % g.cn_e1, col / g.cn_e1,
                                         (int)pw.batch);
                            bulk_commit();
                        }
                        ++n_boxes;
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(leader_promoted0 + 8u * buf);
                    continue;
                }
                float* C = reinterpret_cast<float*>(g.c);
                if (live) C += g.c_b[pw.batch] + g.c_m[pw.tr_m.base + row];
                const float* D = g.mul;  // fused multiplier's row (MUL only)
                if constexpr (MUL)
                    if (live) D += g.d_b[pw.batch] + g.d_m[pw.tr_m.base + row];
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    const TileRows trn = pw.tr_n[h];
                    if (trn.valid <= 0) continue;  // warp-uniform: the whole half lies past the end
                    // closed form of the column offsets (two output modes at most), else the table
                    const bool closed = g.cn_e1 != 0;
                    const int e1 = closed ? g.cn_e1 : 1;
                    const int outer = closed ? (int)(trn.base / e1) : 0;
                    int inner = closed ? (int)(trn.base - (int64_t)outer * e1) : 0;
                    float* p = C + (closed ? inner * g.cn_s1 + outer * g.cn_s2 : 0);
                    const int64_t wrap = g.cn_s2 - (int64_t)e1 * g.cn_s1;
                    const float* d = D + (closed ? inner * g.dn_s1 + outer * g.dn_s2 : 0);
                    const int64_t dwrap = g.dn_s2 - (int64_t)e1 * g.dn_s1;
#pragma unroll 1
                    for (int c0 = 0; c0 < 128 && c0 < trn.valid; c0 += 16) {
                        uint32_t r[16];
                        tc_ld16(tmem_row + (uint32_t)(buf * BN + h * g.half_w + c0), r);
                        float dv[MUL ? 16 : 1];
                        if constexpr (MUL) {
                            // the multiplier's 16 values, all requested before the first store
                            int din = inner;
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                dv[j] = (live && c0 + j < trn.valid) ? (closed ? *d : D[g.d_n[trn.base + c0 + j]]) : 1.f;
                                d += g.dn_s1;
                                if (++din == e1) {
                                    din = 0;
                                    d += dwrap;
                                }
                            }
                        }
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (live && c0 + j < trn.valid) {
                                float* q = closed ? p : C + g.c_n[trn.base + c0 + j];
                                float v = g.alpha * __uint_as_float(r[j]);
                                if constexpr (MUL) v *= dv[j];
                                if (read_c) v += g.beta * *q;
                                *q = v;
                            }
                            p += g.cn_s1;
                            if (++inner == e1) {
                                inner = 0;
                                p += wrap;
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leader_promoted0 + 8u * buf);
            }
            if (lane == 0) bulk_wait<0>();  // every bulk store of this warp has been performed
        }
    } else {
        // ---------------------------------------------------------------- split + promote, then epilogue
        reg_acquire<kWorkerRegs>();
        const int t = threadIdx.x - kLead;
        const int lane_grp = warp & 3;
        const int half = (warp - kLeadWarps) >> 2;  // which half of the tile's columns this warp reads back
        const int col0 = half * CPW;       // its columns in the split-K partials
        const uint32_t tmem_mine = tmem_base + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)(half * g.half_w);
        const uint32_t leader_split0 = map_to_cta(bar_split(0), 0), leader_promoted0 = map_to_cta(bar_promoted(0), 0);
        float acc[CPW];
        uint32_t it = 0, ch0 = 0;  // k-blocks and chunks handled before this work item
        // Deferred epilogue.  All pairs finish their tiles at about the same time, so storing a
        // tile right away makes every SM write at once while every tensor core waits.  The
        // finished sums stay in `acc` instead and leave in kSlices slices, one after each of the
        // next tile's first k-blocks (its first promotion, which needs `acc` cleared, comes
        // later); what is left is flushed before that promotion.
        constexpr int kSlices = 6;
        // With the TMA-store epilogue the pending tile leaves in kTmaSlices boxes of kBoxCols columns,
        // staged in this warp's box of shared memory (worker number = slot) and written by one bulk store each.
        constexpr int kTmaSlices = CPW / kBoxCols;
        const bool c_tma = !MUL && g.c_tma;
        const int n_slices = c_tma ? kTmaSlices : kSlices;
        float* const my_box = out_stage_ptr + (warp - kLeadWarps) * (kBoxBytes / 4) + lane;
        const uint32_t my_box_addr = out_stage + (uint32_t)((warp - kLeadWarps) * kBoxBytes);
        int pend_m_in = 0, pend_m_out = 0, pend_batch = 0;  // tensor-map coordinates of the pending tile's rows
        float* pend_row = nullptr;   // &C[row, 0] of the pending tile, nullptr: nothing pending
        const float* pend_drow = nullptr;  // the fused multiplier's row of that tile, nullptr: no multiplier
        int pend_col0 = 0;           // linear index of its first column
        int pend_valid = 0, pend_next = kSlices;
        auto store_box = [&](int sl) {
            if (kBoxCols * sl >= pend_valid) return;  // warp-uniform: these columns lie past the end
            if (lane == 0) bulk_wait_read<0>();  // the previous box of this warp has been read
            __syncwarp();
            static_assert(kTmaSlices == 4, "the if-chain below names every box of a warp's columns");
            if (sl == 0) stage_acc_cols<0, CPW>(acc, my_box, g.alpha);
            else if (sl == 1) stage_acc_cols<1, CPW>(acc, my_box, g.alpha);
            else if (sl == 2) stage_acc_cols<2, CPW>(acc, my_box, g.alpha);
            else stage_acc_cols<3, CPW>(acc, my_box, g.alpha);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                const int col = pend_col0 + kBoxCols * sl;
                tma_store_5d(&map_c, my_box_addr, pend_m_in, pend_m_out, col % g.cn_e1, col / g.cn_e1, pend_batch);
                bulk_commit();
            }
        };
        auto store_slice_scalar = [&](int sl) {
            // an if-chain on purpose: with a switch the compiler turns the slice number into an
            // index and moves `acc` to local memory
            if (sl == 0) store_acc_slice<0, kSlices, CPW, MUL>(acc, pend_row, pend_col0, g.cn_e1, g.cn_s1, g.cn_s2, pend_valid, g.alpha, g.beta, pend_drow, g.dn_s1, g.dn_s2);
            else if (sl == 1) store_acc_slice<1, kSlices, CPW, MUL>(acc, pend_row, pend_col0, g.cn_e1, g.cn_s1, g.cn_s2, pend_valid, g.alpha, g.beta, pend_drow, g.dn_s1, g.dn_s2);
            else if (sl == 2) store_acc_slice<2, kSlices, CPW, MUL>(acc, pend_row, pend_col0, g.cn_e1, g.cn_s1, g.cn_s2, pend_valid, g.alpha, g.beta, pend_drow, g.dn_s1, g.dn_s2);
            else if (sl == 3) store_acc_slice<3, kSlices, CPW, MUL>(acc, pend_row, pend_col0, g.cn_e1, g.cn_s1, g.cn_s2, pend_valid, g.alpha, g.beta, pend_drow, g.dn_s1, g.dn_s2);
            else if (sl == 4) store_acc_slice<4, kSlices, CPW, MUL>(acc, pend_row, pend_col0, g.cn_e1, g.cn_s1, g.cn_s2, pend_valid, g.alpha, g.beta, pend_drow, g.dn_s1, g.dn_s2);
            else store_acc_slice<5, kSlices, CPW, MUL>(acc, pend_row, pend_col0, g.cn_e1, g.cn_s1, g.cn_s2, pend_valid, g.alpha, g.beta, pend_drow, g.dn_s1, g.dn_s2);
        };
        auto store_slice = [&](int sl) {
            if (c_tma) store_box(sl);
            else store_slice_scalar(sl);
        };
        auto flush_pending = [&]() {
            if (pend_row) {
#pragma unroll
                for (int sl = 0; sl < kSlices; ++sl)
                    if (sl >= pend_next && sl < n_slices) store_slice(sl);
                pend_next = n_slices;
            }
            pend_row = nullptr;
        };
        auto promote = [&](uint32_t chunk) {
            const int buf = chunk & 1;
            if (lane == 0) mbar_wait(bar_chunk(buf), (chunk >> 1) & 1, g.status, 0x114);
            __syncwarp();
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < CPW; c0 += 16) {
                uint32_t r[16];  // 16 columns at a time: the running sums need the registers
                tc_ld16(tmem_mine + (uint32_t)(buf * BN + c0), r);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c0 + j] += __uint_as_float(r[j]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_promoted0 + 8u * buf);
        };
        for (int64_t w = w0; w < n_work; w += wstep) {
        const PairWork pw = pair_work(g, w, rank);
        const int num_kb = pw.num_kb, num_chunks = (num_kb + kChunk - 1) / kChunk;
        const TileRows tr_m = pw.tr_m;
        const int64_t bb = pw.batch;
        auto convert_block = [&]() {
            const int s = it % STAGES;
            const uint32_t use = it / STAGES;
            if (lane == 0) mbar_wait(bar_full(s), use & 1, g.status, 0x113);
            __syncwarp();
            char* big = smem + (size_t)s * Cfg::STAGE_BYTES;
            char* small = big + Cfg::A_BYTES + Cfg::B_BYTES;
            constexpr int CHUNKS = (Cfg::A_BYTES + Cfg::B_BYTES) / 16;
            if constexpr (BF16C) {
                convert_stage_bf16<kSplitThreads>(big, small, t, g.a.mn_major != 0, g.b.mn_major != 0);
            } else {
#pragma unroll 8
                for (int c = t; c < CHUNKS; c += kSplitThreads) {
                    const float4 v = *reinterpret_cast<const float4*>(big + (size_t)c * 16);
                    float4 sm;
                    // raw tile = truncated big operand; remainder exact, rounded to tf32
                    sm.x = remainder_rounded(v.x);
                    sm.y = remainder_rounded(v.y);
                    sm.z = remainder_rounded(v.z);
                    sm.w = remainder_rounded(v.w);
                    *reinterpret_cast<float4*>(small + (size_t)c * 16) = sm;
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_split0 + 8u * s);
            ++it;
        };
        // No promotion of this tile is due before k-block kChunk - 1 + STAGES: until then `acc`
        // still holds the previous tile, which leaves slice by slice.
        constexpr int kQuiet = kChunk - 1 + STAGES;
        static_assert(kQuiet >= kSlices && kQuiet >= kTmaSlices, "every slice gets a k-block of its own");
        int kb = 0;
        for (; kb < num_kb && kb < kQuiet; ++kb) {
            convert_block();
            if (pend_row && pend_next < n_slices) store_slice(pend_next++);
        }
        flush_pending();
#pragma unroll
        for (int j = 0; j < CPW; ++j) acc[j] = 0.f;
        int next_promote = 0;
        for (; kb < num_kb; ++kb) {
            convert_block();
            while (next_promote < num_chunks &&
                   min((next_promote + 1) * kChunk, num_kb) - 1 + STAGES <= kb)
                promote(ch0 + next_promote++);
        }
        while (next_promote < num_chunks) promote(ch0 + next_promote++);
        ch0 += (uint32_t)num_chunks;

        const int row = lane_grp * 32 + lane;
        const TileRows trn = half ? pw.tr_n[1] : pw.tr_n[0];
        if (g.partial) {
            // raw partial sums of this CTA's 128 x 256 part, rows fastest
            float* P = g.partial + ((size_t)((pw.pair_tile * 2 + rank) * g.k_split + pw.split) * BN + col0) * kBM + row;
#pragma unroll
            for (int j = 0; j < CPW; ++j) P[(size_t)j * kBM] = acc[j];
        } else if (c_tma) {
            // the warp's 32 rows x 128 columns leave as boxes during the next tile's first k-blocks
            if (32 * lane_grp < tr_m.valid && trn.valid > 0) {
                const int64_t row_lin = tr_m.base + 32 * lane_grp;
                pend_row = reinterpret_cast<float*>(g.c);  // only marks "pending" on this path
                pend_m_in = (int)(row_lin % g.cm_e1);
                pend_m_out = (int)(row_lin / g.cm_e1);
                pend_batch = (int)bb;
                pend_col0 = (int)trn.base;
                pend_valid = trn.valid;
                pend_next = 0;
            }
        } else if (row < tr_m.valid && trn.valid > 0) {
            float* C = reinterpret_cast<float*>(g.c) + g.c_b[bb] + g.c_m[tr_m.base + row];
            if (g.cn_e1 != 0) {
                // deferred: leaves in slices during the next tile's first k-blocks
                pend_row = C;
                if constexpr (MUL) pend_drow = g.mul + g.d_b[bb] + g.d_m[tr_m.base + row];
                pend_col0 = (int)trn.base;
                pend_valid = trn.valid;
                pend_next = 0;
            } else {
                // columns without a common stride: through the table, right away
                const bool read_c = g.beta != 0.f;
                if constexpr (MUL) {
                    const float* D = g.mul + g.d_b[bb] + g.d_m[tr_m.base + row];
#pragma unroll
                    for (int j = 0; j < CPW; ++j)
                        if (j < trn.valid) acc[j] *= D[g.d_n[trn.base + j]];
                }
#pragma unroll
                for (int j = 0; j < CPW; ++j) {
                    if (j < trn.valid) {
                        float* p = C + g.c_n[trn.base + j];
                        float v = g.alpha * acc[j];
                        if (read_c) v += g.beta * *p;
                        *p = v;
                    }
                }
            }
        }
        }
        flush_pending();
        if (c_tma && lane == 0) bulk_wait<0>();  // every bulk store of this warp has been performed
    }
    tc_fence_before();
    cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still reach into it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    }
}

// Split-K finish for the pair kernel: one CTA per (pair tile, rank), i.e. per 128 x 256 part.
__global__ void __launch_bounds__(256) tf32x3_pair_splitk_finish_kernel(TcArgs g) {
    constexpr int BN = PairCfg::BN;
    const int64_t part = blockIdx.x, pair_tile = part >> 1;
    const int rank = (int)(part & 1);
    const int64_t tiles_mp = (g.tiles_m + 1) / 2, tiles_np = (g.tiles_n + 1) / 2;
    const TileCoord tc = decode_tile(pair_tile, tiles_mp, tiles_np, g.group_m);
    if (2 * tc.tm + rank >= g.tiles_m) return;
    const TileRows tr_m = tile_rows(g.a, 2 * tc.tm + rank, kBM, g.M);
    const int row = threadIdx.x & (kBM - 1);
    if (row >= tr_m.valid) return;
    float* C = reinterpret_cast<float*>(g.c) + g.c_b[tc.batch];
    const int64_t cm = g.c_m[tr_m.base + row];
    const bool read_c = g.beta != 0.f;
    const float* P = g.partial + (size_t)part * g.k_split * BN * kBM + row;
    const float* D = g.mul ? g.mul + g.d_b[tc.batch] + g.d_m[tr_m.base + row] : nullptr;
    // blockIdx.y takes kFinishCols columns of one of the two 128-column halves
    {
        const int h = (int)(blockIdx.y * kFinishCols) / 128, j0 = (int)(blockIdx.y * kFinishCols) % 128;
        if (2 * tc.tn + h >= g.tiles_n) return;
        const TileRows trn = tile_rows(g.b, 2 * tc.tn + h, g.half_w, g.N);
        const int j_end = min(trn.valid, j0 + kFinishCols);
        for (int j = j0 + threadIdx.x / kBM; j < j_end; j += 256 / kBM) {
            float sum = 0.f;
#pragma unroll 8
            for (int s = 0; s < g.k_split; ++s) sum += P[((size_t)s * BN + h * 128 + j) * kBM];
            float* p = C + cm + g.c_n[trn.base + j];
            float v = g.alpha * sum;
            if (D) v *= D[g.d_n[trn.base + j]];
            if (read_c) v += g.beta * *p;
            *p = v;
        }
    }
}

// ------------------------------------------------------------------ operand repack
// Copies one operand, through its offset tables, into a K-major block [batch][row][Kp].  Used
// for large products whose operand TMA cannot describe, or could only tile with mostly
// padding (a free index left with a short extent by sharding): one extra pass over that
// operand is noise next to the product, the exact-FMA fallback is not.
struct RepackArgs {
    const float* src;
    const int64_t* row_tab;
    const int64_t* k_tab;
    const int64_t* b_tab;
    int64_t rows, K, Kp, B;
    int src_kfast;
    float* dst;
};
constexpr int kRepackTile = 64;
__global__ void __launch_bounds__(256) repack_kmajor_kernel(RepackArgs g) {
    constexpr int T = kRepackTile;
    __shared__ float tile[T][T + 1];
    const int64_t tiles_r = (g.rows + T - 1) / T, tiles_k = (g.Kp + T - 1) / T;
    const int64_t n_tiles = tiles_r * tiles_k * g.B;
    const int tx = threadIdx.x & (T - 1), ty = threadIdx.x / T;  // 64 x 4
    constexpr int kPer = T * T / 256;                            // elements per thread and tile
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const int64_t tr = t % tiles_r, rest = t / tiles_r, tk = rest % tiles_k, b = rest / tiles_k;
        const int64_t r0 = tr * T, k0 = tk * T;
        const float* src = g.src + g.b_tab[b];
        // tx runs along the source's fast direction: its offset is looked up once per tile, and the
        // sixteen loads of a thread are all issued before the first one is used
        const int64_t fast = (g.src_kfast ? k0 : r0) + tx;
        const bool fast_ok = g.src_kfast ? fast < g.K : fast < g.rows;
        const int64_t fast_off = fast_ok ? (g.src_kfast ? g.k_tab[fast] : g.row_tab[fast]) : 0;
        float v[kPer];
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int64_t slow = (g.src_kfast ? r0 : k0) + ty + 4 * i;
            const bool ok = fast_ok && (g.src_kfast ? slow < g.rows : slow < g.K);
            v[i] = ok ? src[fast_off + (g.src_kfast ? g.row_tab[slow] : g.k_tab[slow])] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int j = ty + 4 * i;
            if (g.src_kfast) tile[j][tx] = v[i]; else tile[tx][j] = v[i];  // tile[r][k]
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int64_t r = r0 + ty + 4 * i, k = k0 + tx;
            if (r < g.rows && k < g.Kp) g.dst[(b * g.rows + r) * g.Kp + k] = tile[ty + 4 * i][tx];
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// One operand as TMA sees it: a rank-5 tensor [major1, major2, minor1, minor2, batch] where the
// "major" group is the one with the unit stride (K for a K-major tile, the free group for an
// MN-major tile) and every group holds at most two modes.
struct OperandMap {
    bool ok = false;
    TcGeom geom{};
    CUtensorMap map;
};

struct GroupDims {
    int64_t e1 = 1, s1 = 0, e2 = 1, s2 = 0;  // inner / outer extent and stride (elements)
    bool two = false;
};
bool group_dims(const std::vector<Mode>& g, int tns, GroupDims* out) {
    if (g.size() > 2) return false;
    if (g.size() >= 1) { out->e1 = g[0].extent; out->s1 = g[0].s[tns]; }
    if (g.size() == 2) { out->e2 = g[1].extent; out->s2 = g[1].s[tns]; out->two = true; }
    return true;
}

// `free` = the M (or N) group, tns = tensor index (0: A, 1: B), rows = tile rows (128 or BN).
OperandMap make_operand_map(const ContractProblem& p, const std::vector<Mode>& free, int tns, const void* base, int rows) {
    OperandMap out;
    EncodeTiledFn enc = encode_fn();
    if (!enc || p.batch.size() > 1) return out;
    GroupDims f, k;
    if (!group_dims(free, tns, &f) || !group_dims(p.k, tns, &k)) return out;
    if ((uintptr_t)base % 16 != 0) return out;
    const int64_t B = p.batch.empty() ? 1 : p.batch[0].extent, bs = p.batch.empty() ? 0 : p.batch[0].s[tns];
    auto aligned = [](int64_t s) { return s > 0 && s % 4 == 0; };  // 16-byte multiples, positive
    TcGeom& g = out.geom;
    cuuint64_t dims[5], strides[4];
    cuuint32_t box[5] = {1, 1, 1, 1, 1}, estr[5] = {1, 1, 1, 1, 1};
    // Strides of size-1 dimensions are never used for addressing; any 16-byte multiple will do.
    auto stride_or_dummy = [&](int64_t extent, int64_t s) -> int64_t { return extent > 1 ? s : 4; };
    g.e1 = (int)f.e1;
    if (k.s1 == 1 && k.e1 >= 1) {
        // K-major: unit stride on the inner K mode.
        g.mn_major = 0;
        if ((k.two && !aligned(k.s2)) || (f.e1 > 1 && !aligned(f.s1)) || (f.two && f.e2 > 1 && !aligned(f.s2))) return out;
        dims[0] = k.e1; dims[1] = k.e2; dims[2] = f.e1; dims[3] = f.e2; dims[4] = B;
        strides[0] = stride_or_dummy(k.e2, k.s2) * 4;
        strides[1] = stride_or_dummy(f.e1, f.s1) * 4;
        strides[2] = stride_or_dummy(f.e2, f.s2) * 4;
        strides[3] = stride_or_dummy(B, bs) * 4;
        box[0] = kBK;
        if (f.two && f.e1 < rows && rows % f.e1 == 0) {
            g.pack = 1; g.tiles1 = 1;
            box[2] = (cuuint32_t)f.e1; box[3] = (cuuint32_t)(rows / f.e1);
        } else {
            g.pack = 0; g.tiles1 = (int)((f.e1 + rows - 1) / rows);
            box[2] = (cuuint32_t)rows;
        }
    } else if (f.s1 == 1 && f.e1 > 1) {
        // MN-major: unit stride on the inner free mode; boxes are [32 k][32 mn].
        g.mn_major = 1;
        if ((f.two && f.e2 > 1 && !aligned(f.s2)) || (k.e1 > 1 && !aligned(k.s1)) || (k.two && k.e2 > 1 && !aligned(k.s2))) return out;
        dims[0] = f.e1; dims[1] = f.e2; dims[2] = k.e1; dims[3] = k.e2; dims[4] = B;
        strides[0] = stride_or_dummy(f.e2, f.s2) * 4;
        strides[1] = stride_or_dummy(k.e1, k.s1) * 4;
        strides[2] = stride_or_dummy(k.e2, k.s2) * 4;
        strides[3] = stride_or_dummy(B, bs) * 4;
        box[0] = 32; box[2] = kBK;
        if (f.two && f.e1 % 32 == 0) {
            g.pack = 1; g.tiles1 = 1;  // tiles follow the linear row index; each 32-row box is placed on its own
        } else {
            g.pack = 0; g.tiles1 = (int)((f.e1 + rows - 1) / rows);
        }
    } else {
        return out;
    }
    if (B > 1 && !aligned(bs)) return out;
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 != 0 || strides[i] >= (1ull << 40)) return out;
    for (int i = 0; i < 5; ++i)
        if (dims[i] == 0 || dims[i] > 0xffffffffull) return out;
    CUresult r = enc(&out.map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     g.mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    out.ok = (r == CUDA_SUCCESS);
    return out;
}

// The output as a rank-5 tensor [m1, m2, n1, n2, batch] for TMA stores of {32 rows, kBoxCols columns}
// boxes.  `m` / `n` / `batch` are the output's M, N and batch modes in the order the kernel
// linearises rows and columns (the operands' order), with the output's element strides in slot 2;
// `scale` = 2 views a complex output as floats (the unit-stride row mode then holds interleaved
// real and imaginary rows).  Fails (returns false) for layouts a tensor store cannot express; the
// kernel then keeps its per-element stores.
bool make_output_map(void* base, const std::vector<Mode>& m, const std::vector<Mode>& n, const std::vector<Mode>& batch,
                     int scale, const TcGeom& ga, const TcGeom& gb, CUtensorMap* map, int* cm_e1) {
    EncodeTiledFn enc = encode_fn();
    if (!enc || m.empty() || n.empty() || m.size() > 2 || n.size() > 2 || batch.size() > 1) return false;
    if ((uintptr_t)base % 16 != 0 || m[0].s[2] != 1) return false;
    const int64_t e1 = scale * m[0].extent, e2 = m.size() == 2 ? m[1].extent : 1;
    const int64_t s2 = m.size() == 2 ? scale * m[1].s[2] : 4;
    const int64_t f1 = n[0].extent, f2 = n.size() == 2 ? n[1].extent : 1;
    const int64_t t1 = scale * n[0].s[2], t2 = n.size() == 2 ? scale * n[1].s[2] : 4;
    const int64_t B = batch.empty() ? 1 : batch[0].extent, bs = batch.empty() ? 4 : scale * batch[0].s[2];
    auto aligned = [](int64_t extent, int64_t st) { return extent <= 1 || (st > 0 && st % 4 == 0); };
    if (!aligned(e2, s2) || !aligned(f1, t1) || !aligned(f2, t2) || !aligned(B, bs)) return false;
    // A warp's 32 rows (a box's columns) must lie inside one run of the unit-stride row mode (one run
    // of the inner column mode): either the mode is the only one of its group, or the run length
    // is a multiple of the box, or the kernel's tiles never cross a run (tiling inside the inner
    // mode of a two-mode group, the same mode here).
    const bool rows_ok = m.size() == 1 || e1 % 32 == 0 || (!ga.pack && ga.e1 == e1 && scale == 1);
    const bool cols_ok = n.size() == 1 || f1 % kBoxCols == 0 || (!gb.pack && gb.e1 == f1);
    if (!rows_ok || !cols_ok) return false;
    if (e1 >= INT32_MAX || f1 >= INT32_MAX) return false;
    auto stride_or_dummy = [](int64_t extent, int64_t st) -> cuuint64_t { return (cuuint64_t)(extent > 1 ? st : 4) * 4; };
    cuuint64_t dims[5] = {(cuuint64_t)e1, (cuuint64_t)e2, (cuuint64_t)f1, (cuuint64_t)f2, (cuuint64_t)B};
    cuuint64_t strides[4] = {stride_or_dummy(e2, s2), stride_or_dummy(f1, t1), stride_or_dummy(f2, t2), stride_or_dummy(B, bs)};
    cuuint32_t box[5] = {32, 1, kBoxCols, 1, 1}, estr[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 != 0 || strides[i] >= (1ull << 40)) return false;
    for (int i = 0; i < 5; ++i)
        if (dims[i] == 0 || dims[i] > 0xffffffffull) return false;
    if (enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    *cm_e1 = (int)e1;
    return true;
}

// Split K when the tiles alone leave SMs idle: pick the split that minimises
// (waves of CTAs) x (k-blocks per CTA + a fixed cost for prologue, epilogue and the finishing
// pass), preferring fewer splits unless more of them save a tenth.  `slots` = tiles that run at once.
void choose_k_split(TcArgs* g, int64_t n_tiles, int64_t slots) {
    g->k_split = 1;
    g->kb_per_split = g->num_kb;
    const int want = env_int("TFB_TC_KSPLIT", 0);
    auto cost = [&](int ksp, int* per) {
        const int kbp = (g->num_kb + ksp - 1) / ksp, real = (g->num_kb + kbp - 1) / kbp;
        *per = kbp;
        return (double)((n_tiles * real + slots - 1) / slots) * (kbp + 8.0) + (real > 1 ? 4.0 : 0.0);
    };
    int best = 1, per = g->num_kb;
    double best_cost = cost(1, &per);
    if (want > 1) {
        best = std::min(want, std::max(1, g->num_kb / kChunk));
    } else if (want == 0) {
        const int max_split = std::min(64, g->num_kb / kChunk);
        for (int ksp = 2; ksp <= max_split; ++ksp) {
            const double c = cost(ksp, &per);
            if (c < 0.9 * best_cost) { best = ksp; best_cost = c; }
        }
    }
    if (best > 1) {
        cost(best, &per);
        g->kb_per_split = per;
        g->k_split = (g->num_kb + per - 1) / per;
    }
}

template <int BN>
tfb_status launch_tc(tfb_ctx* ctx, const OperandMap& a, const OperandMap& b, TcArgs g) {
    using Cfg = TcCfg<BN>;
    static std::mutex mu;
    static std::map<int, bool> configured;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[ctx->device]) {
            TFB_CUDA(cudaFuncSetAttribute(contract_tf32x3_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          Cfg::SMEM_BYTES));
            configured[ctx->device] = true;
        }
    }
    g.a = a.geom;
    g.b = b.geom;
    auto tiles = [](const TcGeom& o, int64_t total, int rows) -> int64_t {
        if (o.pack) return (total + rows - 1) / rows;
        return (total / o.e1) * o.tiles1;  // outer extent x tiles per inner slice
    };
    g.tiles_m = tiles(g.a, g.M, kBM);
    g.tiles_n = tiles(g.b, g.N, BN);
    g.group_m = env_int("TFB_TC_GROUP_M", 16);
    const int64_t n_tiles = g.tiles_m * g.tiles_n * g.B;
    choose_k_split(&g, n_tiles, ctx->sm_count);
    const int64_t grid = n_tiles * g.k_split;
    if (grid > 0x7fffffff) return fail(TFB_ERR_INVALID_ARGUMENT, "contraction too large for one launch");
    PoolBlock ws;
    if (g.k_split > 1) {
        TFB_TRY(ws.alloc(ctx, (size_t)grid * BN * kBM * sizeof(float)));
        g.partial = (float*)ws.ptr;
    }
    {
        LaunchScope ls(ctx, "contract_tf32x3");
        contract_tf32x3_kernel<BN><<<(unsigned)grid, 64 + kSplitThreads, Cfg::SMEM_BYTES, ctx->stream>>>(a.map, b.map, g);
        TFB_CUDA(cudaGetLastError());
    }
    if (g.k_split > 1) {
        LaunchScope ls(ctx, "contract_tf32x3_finish");
        tf32x3_splitk_finish_kernel<BN><<<dim3((unsigned)n_tiles, BN / kFinishCols), 256, 0, ctx->stream>>>(g);
        TFB_CUDA(cudaGetLastError());
    }
    return TFB_OK;
}

tfb_status launch_tc_pair(tfb_ctx* ctx, const OperandMap& a, const OperandMap& b, const CUtensorMap* c_map, TcArgs g) {
    using Cfg = PairCfg;
    static std::mutex mu;
    static std::map<int, bool> configured;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[ctx->device]) {
#define TFB_PAIR_SMEM(MUL_, SHORT_, C_)                                                                    \
    TFB_CUDA(cudaFuncSetAttribute(contract_tf32x3_pair_kernel<MUL_, SHORT_, C_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  Cfg::SMEM_BYTES))
            TFB_PAIR_SMEM(false, false, false);
            TFB_PAIR_SMEM(true, false, false);
            TFB_PAIR_SMEM(false, true, false);
            TFB_PAIR_SMEM(true, true, false);
            TFB_PAIR_SMEM(false, true, true);
            TFB_PAIR_SMEM(true, true, true);
            TFB_PAIR_SMEM(false, false, true);
            TFB_PAIR_SMEM(true, false, true);
#undef TFB_PAIR_SMEM
            configured[ctx->device] = true;
        }
    }
    g.a = a.geom;
    g.b = b.geom;
    auto tiles = [](const TcGeom& o, int64_t total, int rows) -> int64_t {
        if (o.pack) return (total + rows - 1) / rows;
        return (total / o.e1) * o.tiles1;
    };
    g.tiles_m = tiles(g.a, g.M, kBM);  // 128-row tiles; a pair takes two of each
    if (g.half_w == 0) g.half_w = 128;
    g.tiles_n = tiles(g.b, g.N, g.half_w);
    g.group_m = env_int("TFB_TC_GROUP_M", 8);
    const int64_t pair_tiles = ((g.tiles_m + 1) / 2) * ((g.tiles_n + 1) / 2) * g.B;
    choose_k_split(&g, pair_tiles, ctx->sm_count / 2);
    const int64_t n_work = pair_tiles * g.k_split;
    if (2 * n_work > 0x7fffffff) return fail(TFB_ERR_INVALID_ARGUMENT, "contraction too large for one launch");
    // one CTA per SM, so at most sm_count / 2 pairs run at once; each walks the work list with that stride
    const int64_t grid = 2 * std::min<int64_t>(n_work, std::max(1, ctx->sm_count / 2));
    PoolBlock ws;
    const bool via_partials = g.k_split > 1;
    if (via_partials) {
        TFB_TRY(ws.alloc(ctx, (size_t)(2 * n_work) * Cfg::BN * kBM * sizeof(float)));
        g.partial = (float*)ws.ptr;
    }
    // Split-K partials leave through the finishing kernel; a fused multiplier through the scalar path.
    if (via_partials || g.mul || !c_map) g.c_tma = 0;
    const CUtensorMap& mc = (g.c_tma && c_map) ? *c_map : a.map;  // unused when c_tma is off
    {
        LaunchScope ls(ctx, "contract_tf32x3");
        // the cluster shape (2, 1, 1) is a compile-time attribute of the kernel
        // short K, one accumulation chunk per tile: the variant with dedicated drain warps
        const bool short_k = !via_partials && g.num_kb <= kChunk && env_int("TFB_TC_SHORTK", 1);
        // the two correction terms of 3xTF32 as one bf16 MMA (see convert_stage_bf16); a short-K tile of fewer
        // than six k-blocks is dominated by its start and end and keeps the three TF32 MMAs
        const bool bf16c = env_int("TFB_TC_BF16_CORRECTIONS", 1) != 0 && (!short_k || g.num_kb >= 6);
#define TFB_PAIR_LAUNCH(MUL_, SHORT_, C_)                                                                                   \
    contract_tf32x3_pair_kernel<MUL_, SHORT_, C_><<<(unsigned)grid, pair_threads(SHORT_), Cfg::SMEM_BYTES, ctx->stream>>>(a.map, b.map, \
                                                                                                                       mc, g)
#define TFB_PAIR_LAUNCH2(MUL_, SHORT_)                                                                                      \
    do {                                                                                                                    \
        if (bf16c) TFB_PAIR_LAUNCH(MUL_, SHORT_, true);                                                                     \
        else TFB_PAIR_LAUNCH(MUL_, SHORT_, false);                                                                          \
    } while (0)
        if (g.mul && short_k) TFB_PAIR_LAUNCH2(true, true);
        else if (g.mul) TFB_PAIR_LAUNCH2(true, false);
        else if (short_k) TFB_PAIR_LAUNCH2(false, true);
        else TFB_PAIR_LAUNCH2(false, false);
#undef TFB_PAIR_LAUNCH2
#undef TFB_PAIR_LAUNCH
        TFB_CUDA(cudaGetLastError());
    }
    if (via_partials) {
        LaunchScope ls(ctx, "contract_tf32x3_finish");
        tf32x3_pair_splitk_finish_kernel<<<dim3((unsigned)(2 * pair_tiles), Cfg::BN / kFinishCols), 256, 0, ctx->stream>>>(g);
        TFB_CUDA(cudaGetLastError());
    }
    return TFB_OK;
}

// Peak probe: one CTA per SM issues 128 x 256 x 8 TF32 MMAs back to back on operand tiles
// that stay in shared memory; nothing else runs.  The quotient is the dense TF32 rate the
// tensor pipe sustains, the denominator for "fraction of TF32 peak" (a 3xTF32 contraction
// can reach a third of it in algorithmic flops).
__global__ void __launch_bounds__(128, 1) probe_tf32_kernel(int iters, int* status) {
    extern __shared__ char smem_raw[];
    char* smem = (char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t base = smem_u32(smem);
    const uint32_t a_tile = base, b_tile = base + 16384, bar = base + 16384 + 32768, tmem_word = bar + 8;
    // Operand values in (-1, 1) from a hash of the position: what the tensor cores draw depends on
    // how many bits toggle, and constant tiles would let a long run keep a clock that real data
    // (under the board's power limit) does not.
    for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15;
        h *= 2246822519u;
        h ^= h >> 13;
        ((float*)smem)[i] = (float)(int)(h & 0xffffu) * (1.0f / 32768.0f) - 1.0f;
    }
    fence_async_smem();
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(tmem_word, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *(volatile uint32_t*)(smem + 16384 + 32768 + 8);
    if (threadIdx.x == 0) {
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                tc_mma_tf32(tmem_d, smem_desc(a_tile + ks * 32, 16, 1024, 2), smem_desc(b_tile + ks * 32, 16, 1024, 2),
                            idesc, (it | ks) != 0);
        }
        tc_commit(bar);
        mbar_wait(bar, 0, status, 0x201);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_d, 256);
    }
}

}  // namespace

extern "C" tfb_status tfb_probe_tf32_tflops(tfb_ctx* ctx, double* tflops) {
    if (!ctx || !tflops) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_probe_tf32_tflops: NULL argument");
    DeviceGuard g(ctx->device);
    const int smem = 16384 + 32768 + 64 + 1024;
    TFB_CUDA(cudaFuncSetAttribute(probe_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaEvent_t e0, e1;
    TFB_CUDA(cudaEventCreate(&e0));
    TFB_CUDA(cudaEventCreate(&e1));
    const int iters = 20000;
    double best = 0;
    for (int rep = 0; rep < 4; ++rep) {
        TFB_CUDA(cudaEventRecord(e0, ctx->stream));
        probe_tf32_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(iters, ctx->dev_status);
        TFB_CUDA(cudaEventRecord(e1, ctx->stream));
        TFB_CUDA(cudaEventSynchronize(e1));
        float ms = 0;
        TFB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        const double flop = (double)ctx->sm_count * iters * 4 * (2.0 * 128 * 256 * 8);
        const double t = flop / (ms * 1e-3) / 1e12;
        if (rep > 0 && t > best) best = t;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *tflops = best;
    return TFB_OK;
}

// The same probe launched back to back for `seconds`: the rate of the last quarter of the run,
// i.e. what the tensor pipe sustains once the power limit has pulled the clock down.  This is
// the denominator for a kernel timed inside a long step; the burst figure above is the one for
// a kernel timed alone.
extern "C" tfb_status tfb_probe_tf32_tflops_sustained(tfb_ctx* ctx, double seconds, double* tflops) {
    if (!ctx || !tflops) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_probe_tf32_tflops_sustained: NULL argument");
    if (!(seconds > 0) || seconds > 30) return fail(TFB_ERR_INVALID_ARGUMENT, "seconds must be in (0, 30]");
    DeviceGuard g(ctx->device);
    const int smem = 16384 + 32768 + 64 + 1024;
    TFB_CUDA(cudaFuncSetAttribute(probe_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaEvent_t e0, e1;
    TFB_CUDA(cudaEventCreate(&e0));
    TFB_CUDA(cudaEventCreate(&e1));
    const int iters = 20000, batch = 16;
    const double flop_batch = (double)batch * ctx->sm_count * iters * 4 * (2.0 * 128 * 256 * 8);
    std::vector<double> batch_ms;
    double total_ms = 0;
    tfb_status st = TFB_OK;
    while (total_ms < seconds * 1e3 && batch_ms.size() < 4096) {
        cudaEventRecord(e0, ctx->stream);
        for (int i = 0; i < batch; ++i) probe_tf32_kernel<<<ctx->sm_count, 128, smem, ctx->stream>>>(iters, ctx->dev_status);
        cudaEventRecord(e1, ctx->stream);
        float ms = 0;
        if (cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess || ms <= 0) {
            st = fail(TFB_ERR_DEVICE, "tfb_probe_tf32_tflops_sustained: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        batch_ms.push_back(ms);
        total_ms += ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (st != TFB_OK) return st;
    const size_t tail = std::max<size_t>(1, batch_ms.size() / 4);
    double ms_tail = 0;
    for (size_t i = batch_ms.size() - tail; i < batch_ms.size(); ++i) ms_tail += batch_ms[i];
    *tflops = flop_batch * tail / (ms_tail * 1e-3) / 1e12;
    return TFB_OK;
}

// `c_tables`, when given, are device offset tables {batch, row, column} (in floats) that replace
// the ones derived from p's output strides: the complex path writes into a complex tensor
// through its f32 view this way; `c_n_modes` / `c_scale` then describe the column offsets in closed form
// (the N modes of the complex problem, strides times 2).
// set while contract_tcgen05 runs the same product with its operands' roles exchanged
static thread_local bool role_exchanged = false;

tfb_status contract_tcgen05(tfb_ctx* ctx, const ContractProblem& p, bool* declined, const int64_t* const* c_tables,
                            const std::vector<Mode>* c_n_modes, int c_scale, const std::vector<Mode>* c_m_modes,
                            const std::vector<Mode>* c_batch_modes) {
    const std::vector<Mode>* cn_modes = c_tables ? c_n_modes : &p.n;
    const std::vector<Mode>* cm_modes = c_tables ? c_m_modes : &p.m;
    const std::vector<Mode>* cb_modes = c_tables ? c_batch_modes : &p.batch;
    if (!c_tables) c_scale = 1;
    *declined = true;
    if (p.dtype != TFB_F32) return TFB_OK;
    if (env_int("TFB_NO_TCGEN05", 0)) return TFB_OK;
    // Small problems stay on the SIMT kernel: a 128-row tile would be mostly padding.
    if (p.M() < 32 || p.N() < 32 || p.K() < 8) return TFB_OK;
    if (p.M() > INT32_MAX - 256 || p.N() > INT32_MAX - 256 || p.K() > INT32_MAX - 64) return TFB_OK;
    // A narrow output: the short free side becomes the COLUMNS of a single tile (below), whose MMAs
    // then have exactly that many columns.  Which operand supplies rows and which columns is a
    // matter of names - the product is described by modes - so the operands exchange roles when
    // the short side is the first one's.
    if (!role_exchanged && p.M() <= 256 && p.N() > 256 && p.m.size() == 1 && !p.mul && env_int("TFB_TC_NARROW", 1) &&
        env_int("TFB_TC_PAIR", 1)) {
        const ContractProblem q = exchange_roles(p);
        const int64_t* swapped[3] = {c_tables ? c_tables[0] : nullptr, c_tables ? c_tables[2] : nullptr,
                                     c_tables ? c_tables[1] : nullptr};
        role_exchanged = true;
        // With offset tables from the caller (the Complex32 embedding) the new columns are the caller's
        // rows, which only its table describes: no closed form for them and no tensor-store map.
        const tfb_status st = c_tables ? contract_tcgen05(ctx, q, declined, swapped, nullptr, c_scale, nullptr, c_batch_modes)
                                       : contract_tcgen05(ctx, q, declined);
        role_exchanged = false;
        return st;
    }
    const int64_t M = p.M(), N = p.N(), K = p.K();
    // Up to 256 columns in all, one unfused column mode, more rows than one CTA takes: one pair tile
    // of 2 * half_w columns (see TcArgs::half_w).
    int half_w = 0;
    if (N <= 256 && M > kBM && p.n.size() == 1 && env_int("TFB_TC_NARROW", 1) && env_int("TFB_TC_PAIR", 1))
        half_w = (int)((N + 63) / 64) * 32;
    const int bn = half_w ? 256 : (N >= 256 && env_int("TFB_TC_BN", 256) == 256) ? 256 : 128;
    // Pairs of CTAs on 256 x 256 tiles when the output has room for them.
    const bool pair = half_w || (bn == 256 && M > kBM && env_int("TFB_TC_PAIR", 1));
    const int rows_b = pair ? 128 : bn;
    OperandMap a = make_operand_map(p, p.m, 0, p.a, kBM);
    OperandMap b = make_operand_map(p, p.n, 1, p.b, rows_b);
    // half-tiles of half_w columns: the boxes stay 128 rows tall (what lies past a half is not used)
    auto narrow = [&](OperandMap* o) {
        if (half_w && o->ok && !o->geom.pack) o->geom.tiles1 = (int)((o->geom.e1 + half_w - 1) / half_w);
    };
    narrow(&b);
    std::shared_ptr<ContractTables> t;
    PoolBlock packed_a, packed_b;
    // Large products only: repack an operand that has no tensor map, or whose tiles would be
    // more than a third padding.
    if (!c_tables && 2.0 * M * N * K >= 1e9 && p.batch.size() <= 1 && p.k.size() <= 2) {
        auto wasteful = [](const OperandMap& o, int64_t total, int rows) {
            if (!o.ok) return true;
            if (o.geom.pack) return false;
            return (total / o.geom.e1) * o.geom.tiles1 * rows > total + total / 2;
        };
        const int force_pack = env_int("TFB_TC_REPACK", 0);  // bit 0: A, bit 1: B (experiments)
        bool pack_a = wasteful(a, M, kBM) || (force_pack & 1), pack_b = wasteful(b, N, half_w ? half_w : rows_b) || (force_pack & 2);
        // An MN-major operand of a large product is also worth one pass: with the corrections as a bf16
        // MMA the pair kernel converts K-major tiles faster (8192^3 with N(0,1) operands: 296 against
        // 276 TFLOP/s with A MN-major, 270 with both), the copy runs at 1.9 TB/s, and what it costs is
        // proportional to the operand while what it saves is proportional to the product: from about
        // 5000 rows of the OTHER operand on the copy is the cheaper side, and at 8192 it nets 5 %.
        // Optional: without room for the copy the product runs on the operand as it lies.
        const bool favour_kmajor = pair && K >= 512 && env_int("TFB_TC_BF16_CORRECTIONS", 1) != 0 && env_int("TFB_TC_REPACK_MN", 1);
        // (a copy of at most an eighth of the device's memory: a larger one could take the room that
        // the caller's next tensors need)
        const double copy_cap = (double)ctx->total_mem / 8 / sizeof(float);
        const bool opt_a = !pack_a && favour_kmajor && a.ok && a.geom.mn_major && N >= 8192 && (double)M * K * p.B() <= copy_cap;
        const bool opt_b = !pack_b && favour_kmajor && b.ok && b.geom.mn_major && M >= 8192 && (double)N * K * p.B() <= copy_cap;
        pack_a |= opt_a;
        pack_b |= opt_b;
        if (pack_a || pack_b) {
            TFB_TRY(get_tables(ctx, p, &t));
            ContractArgs ca;
            fill_args(p, *t, &ca);
            const int64_t Kp = (K + 3) / 4 * 4, Bn = p.B();
            auto repack = [&](int tns, PoolBlock* blk, OperandMap* out) -> tfb_status {
                const int64_t rows = tns == 0 ? M : N;
                const tfb_status got = blk->alloc(ctx, (size_t)(rows * Kp * Bn) * sizeof(float));
                if (got != TFB_OK) {
                    if (tns == 0 ? opt_a : opt_b) return TFB_OK;  // no room for a copy that only saves time
                    return got;
                }
                RepackArgs r{(const float*)(tns == 0 ? p.a : p.b), tns == 0 ? t->a_m : t->b_n, tns == 0 ? t->a_k : t->b_k,
                             tns == 0 ? t->a_b : t->b_b, rows, K, Kp, Bn, tns == 0 ? ca.a_kfast : ca.b_kfast, (float*)blk->ptr};
                const int64_t n_tiles = ((rows + kRepackTile - 1) / kRepackTile) * ((Kp + kRepackTile - 1) / kRepackTile) * Bn;
                {
                    LaunchScope ls(ctx, "repack_operand");
                    repack_kmajor_kernel<<<(unsigned)std::min<int64_t>(n_tiles, (int64_t)ctx->sm_count * 16), 256, 0, ctx->stream>>>(r);
                    TFB_CUDA(cudaGetLastError());
                }
                // the same product with this operand contiguous: one free mode, K split as in the other operand
                ContractProblem q = p;
                std::vector<Mode> free_q{Mode{rows, {0, 0, 0}}};
                free_q[0].s[tns] = Kp;
                int64_t run = 1;
                for (Mode& m : q.k) { m.s[tns] = run; run *= m.extent; }
                for (Mode& m : q.batch) m.s[tns] = rows * Kp;
                *out = make_operand_map(q, free_q, tns, blk->ptr, tns == 0 ? kBM : rows_b);
                return TFB_OK;
            };
            if (pack_a) TFB_TRY(repack(0, &packed_a, &a));
            if (pack_b) {
                TFB_TRY(repack(1, &packed_b, &b));
                narrow(&b);
            }
        }
    }
    if (!a.ok || !b.ok) return TFB_OK;
    TcArgs g;
    memset(&g, 0, sizeof g);
    g.c = (char*)p.c;
    // closed form of the output's column offsets (in floats; `c_scale` = 2 for the f32 view of a complex output)
    g.cn_e1 = 0;
    if (cn_modes && !cn_modes->empty() && cn_modes->size() <= 2 && (*cn_modes)[0].extent < INT32_MAX) {
        const std::vector<Mode>& nm = *cn_modes;
        g.cn_e1 = nm.size() == 2 ? (int)nm[0].extent : INT32_MAX;
        g.cn_s1 = c_scale * nm[0].s[2];
        g.cn_s2 = nm.size() == 2 ? c_scale * nm[1].s[2] : 0;
        g.dn_s1 = nm[0].s[3];
        g.dn_s2 = nm.size() == 2 ? nm[1].s[3] : 0;
    }
    if (c_tables) {
        g.c_b = c_tables[0]; g.c_m = c_tables[1]; g.c_n = c_tables[2];
    } else {
        if (!t) TFB_TRY(get_tables(ctx, p, &t));
        g.c_b = t->c_b; g.c_m = t->c_m; g.c_n = t->c_n;
    }
    if (p.mul) {
        if (!t) TFB_TRY(get_tables(ctx, p, &t));
        g.mul = (const float*)p.mul;
        g.d_b = t->d_b; g.d_m = t->d_m; g.d_n = t->d_n;
    }
    g.M = M; g.N = N; g.K = K; g.B = p.B();
    g.half_w = half_w ? half_w : 128;
    g.alpha = (float)p.alpha.re;
    g.beta = (float)p.beta.re;
    // Both operands walk K in the same blocks: 32 at a time inside the inner K mode.
    g.k_e1 = (int)p.k[0].extent;
    g.k_blocks1 = (g.k_e1 + kBK - 1) / kBK;
    g.num_kb = (int)((K / g.k_e1) * g.k_blocks1);
    g.status = ctx->dev_status;
    *declined = false;
    // Output through TMA stores where the layout allows it and nothing of the old output is needed.
    CUtensorMap c_map;
    bool have_c_map = false;
    if (pair && g.beta == 0.f && !p.mul && g.cn_e1 != 0 && cm_modes && cn_modes && cb_modes &&
        env_int("TFB_TC_TMA_STORE", 1)) {
        int cm_e1 = 0;
        have_c_map = make_output_map(p.c, *cm_modes, *cn_modes, *cb_modes, c_scale, a.geom, b.geom, &c_map, &cm_e1);
        if (have_c_map) {
            g.c_tma = 1;
            g.cm_e1 = cm_e1;
        }
    }
    if (pair) return launch_tc_pair(ctx, a, b, have_c_map ? &c_map : nullptr, g);
    return bn == 256 ? launch_tc<256>(ctx, a, b, g) : launch_tc<128>(ctx, a, b, g);
}

}  // namespace tfb
