// Grouped f32 products on the tcgen05 tensor cores: the kernel of tfb_grouped_gemm for ragged
// tables of column-major problems that the mma.sync kernel (grouped_tf32.cu) declines - any
// m, n, k >= 1 with 16-byte aligned columns and K up to 512 - where it is about five times as
// fast as the SIMT kernel (4096 problems with dims from {20, 36, 72, 136}: 174 us against 832).
// On tables the mma.sync kernel takes (dims in multiples of 16, K <= 128) that kernel is the
// faster one (54 us against 96 for 4096 problems with dims from {16, 32, 64, 128}); see the end of
// this comment for why.  TFB_GROUPED_PREFER_TCGEN05=1 asks for this kernel first.
//
//   * a unit is a 128 x 128 output tile of one problem (most problems are one unit), a STAGE is
//     at most 32 of its K; one persistent CTA per SM runs the stage sequence the host laid out
//     for it (64-byte records, longest units first, greedily balanced over the CTAs); a warp
//     keeps the next 64 - 128 records in shared memory, so no role waits for a record;
//   * four loader warps copy a stage's operands with 16-byte cp.async straight into the tensor
//     core's swizzled layouts - A, whose rows are contiguous in memory, as [32 k][32 m] boxes
//     (MN-major, 128-byte rows swizzled in 32-byte units), B as [n][32 k] rows (K-major,
//     swizzled in 16-byte units) - with zero fill for whatever lies outside the problem, and
//     hand the stage over through an mbarrier that counts the copies' completion;
//   * stages live in a 216 KB ring whose byte offsets the host planned, so a 3 KB stage takes
//     3 KB and not a fixed slot: every record names the newest earlier stages whose bytes it
//     overwrites, and the loaders wait for exactly those stages' MMAs;
//   * 3xTF32: the tensor core reads the upper 19 bits of the raw words as the "big" parts; four
//     converter warps write the rounded remainders beside them; four threads, each with the
//     units u = i mod 4 and one of four 128-column TMEM accumulators, issue
//     small x big + big x small + big x big per 8-deep k-step; four epilogue warps read
//     finished accumulators and store whole 128-byte column segments while the next units' MMAs run.
// Every wait is bounded (ptx_sm100.cuh): when one expires the kernel records a status word,
// stops waiting everywhere else and ends; tfb_ctx_synchronize reports it.
//
// What bounds it (CUDA events, clock64 traces of one CTA, a tcgen05.mma issue probe):
//   * shared-memory bandwidth.  A stage's bytes cross shared memory six times - written by
//     cp.async, read and written by the converters, read three times by the MMAs - and a
//     128 x 128 x 8 TF32 MMA from shared memory already needs the full 128 bytes per clock (8 KB
//     in 64 cycles).  A 128 x 128 x 32 stage is 192 KB of shared-memory traffic = 1536 clocks, more
//     than its 1350 clocks of HBM time at an SM's share of the bandwidth; the MMA reads all 128
//     rows of the A side whatever m is, so small problems pay for rows they do not have.
//   * instruction issue.  A tcgen05.mma costs its issuing thread 55 - 110 clocks whatever its shape
//     (K is 8 per instruction: 12 instructions per stage), a warp's cp.async or conversion
//     sequence for one stage is a dependent chain of about a thousand clocks.
//   * TMA does not help: every problem needs its own two tensor maps, and fetching a map costs
//     the SM's copy engine about half a microsecond, one map after another (the same kernel
//     with TMA loads: 73 us, 47 of them with the conversion, the MMAs and the stores switched off).
//
// Semantics: C_p = alpha * A_p B_p + beta * C_p per problem, the formula of
// PrimDescriptor::BatchedGemm (tenferro-prims/src/lib.rs:156-168).
#include <algorithm>
#include <deque>
#include <queue>

#include "common.h"
#include "contract_common.cuh"
#include "ptx_sm100.cuh"

namespace tfb {

namespace {

constexpr int kTile = 128;           // unit rows and columns
constexpr int kDepth = 32;           // K per stage: one 128-byte swizzle row
constexpr int kSlots = 32;           // barrier sets; at most this many stages are in flight
constexpr int kRingBytes = 216 * 1024;
constexpr int kRecords = 128;        // records held in shared memory: two halves, refilled in turn
constexpr int kRecBytes = kRecords * 64;
constexpr int kBarBytes = 1024;
constexpr int kSmemBytes = kRingBytes + kRecBytes + kBarBytes + 1024;  // + slack to align the ring to a swizzle atom
constexpr int kMaxK = 512;           // longest accumulation chain left to the tensor core's truncating adds
constexpr int kLoadWarps = 4, kMmaWarps = 4, kConvWarps = 4, kEpiWarps = 4;
constexpr int kMmaWarp = kLoadWarps;  // warps: loaders, the MMA issuers, converters, epilogue, the record fetcher
constexpr int kConvWarp = kMmaWarp + kMmaWarps, kEpiWarp = kConvWarp + kConvWarps;
constexpr int kRoleWarps = kEpiWarp + kEpiWarps;
constexpr int kThreads = 32 * (kRoleWarps + 1);

enum : uint16_t { kFirst = 1, kLast = 2, kEnd = 4 };

// One stage, 64 bytes, read in 16-byte parts: every role fetches only what it needs.
struct __align__(16) TcStage {
    // part 0: what the converter and the MMA thread need
    uint8_t off_kb, raw_kb;  // ring offset and bytes of the raw operands, in KB; the remainders follow the raw bytes
    uint8_t na, kt;          // [32 k][32 m] boxes of A; 8-deep k-steps with data
    uint16_t mt, nt;         // rows and columns of the unit inside the problem
    uint16_t flags, n_mma;   // flags: kFirst | kLast | kEnd, and the k of this stage that exist (1..32) << 8;
                             // n_mma: nt rounded up to the MMA's granule of 16
    // Before this stage is loaded, the MMAs of the stages whose bytes it overwrites must have
    // finished.  Each of the four MMA issuers (unit number mod 4) finishes its stages in order, so
    // the record names the newest such stage of each issuer (-1: none).
    int32_t dep0;
    // part 1: the unit's corner of each operand at the stage's first k
    const float* a;  // A[m, k] at a + m + k * a_cs
    const float* b;  // B[k, n] at b + k + n * b_cs
    // part 2
    int32_t a_cs, b_cs, c_cs;
    int32_t dep1;
    // part 3
    float* c;  // C[m, n] at c + m + n * c_cs
    int32_t dep2, dep3;
};
static_assert(sizeof(TcStage) == 64, "records are read as four 16-byte parts");

struct GtArgs {
    const TcStage* stages;  // CTA c runs stages[c * pitch + 0, 1, ...] up to its kEnd record
    int pitch;
    float alpha, beta;
    int* status;
};

__device__ __forceinline__ uint4 ld_part(const TcStage* rec, int part) {
    return __ldg(reinterpret_cast<const uint4*>(rec) + part);
}
// A role's window on its CTA's records.  The records sit in shared memory, 64 at a time in each
// of two halves that one warp refills from global memory as soon as every role has left them:
// no role ever waits for a record to come from global memory, which for the single threads that
// issue the MMAs would be a round trip per stage.  The whole warp calls enter(s) before it reads
// record s, for s = 0, 1, 2, ...
struct Records {
    const uint4* recs;
    uint32_t bar_full0, bar_free0;
    int lane;
    int* status;
    __device__ __forceinline__ void enter(uint32_t s) {
        if ((s & 63u) == 0) {
            const uint32_t h = s >> 6;
            __syncwarp();
            if (lane == 0) {
                if (h > 0) mbar_arrive(bar_free0 + 8u * ((h - 1) & 1u));
                mbar_wait(bar_full0 + 8u * (h & 1u), (h >> 1) & 1u, status, 0x306);
            }
            __syncwarp();
        }
    }
    __device__ __forceinline__ uint4 part(uint32_t s, int p) const { return recs[(s & (kRecords - 1)) * 4 + p]; }
};

// 16 bytes global -> shared, the last 16 - bytes of them zero (bytes = 0: nothing is read).
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// This thread's arrival on `bar` happens when all its earlier cp.async have landed; the barrier's
// count has to include it.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46) | ((uint64_t)layout << 61);
}
// a - trunc_tf32(a), exact in f32, plus half a TF32 ulp so that the tensor core's truncation rounds it.
__device__ __forceinline__ float remainder_rounded(float a) {
    const float r = a - __uint_as_float(__float_as_uint(a) & 0xffffe000u);
    return __uint_as_float(__float_as_uint(r) + 0x1000u);
}
__device__ __forceinline__ float4 remainder4(float4 v) {
    return make_float4(remainder_rounded(v.x), remainder_rounded(v.y), remainder_rounded(v.z), remainder_rounded(v.w));
}

__global__ void __launch_bounds__(kThreads, 1) grouped_tc_kernel(GtArgs g) {
    extern __shared__ char smem_raw[];
    char* smem = (char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t ring = smem_u32(smem);
    const uint32_t bars = ring + kRingBytes + kRecBytes;
    auto bar_full = [&](uint32_t s) { return bars + 8u * s; };
    auto bar_conv = [&](uint32_t s) { return bars + 8u * (kSlots + s); };
    auto bar_empty = [&](uint32_t s) { return bars + 8u * (2 * kSlots + s); };
    auto bar_acc_full = [&](uint32_t a) { return bars + 8u * (3 * kSlots + a); };
    auto bar_acc_free = [&](uint32_t a) { return bars + 8u * (3 * kSlots + 4 + a); };
    auto bar_rec_full = [&](uint32_t h) { return bars + 8u * (3 * kSlots + 8 + h); };
    auto bar_rec_free = [&](uint32_t h) { return bars + 8u * (3 * kSlots + 10 + h); };
    const uint32_t tmem_word = bars + 8u * (3 * kSlots + 12);
    volatile uint32_t* tmem_word_ptr = (volatile uint32_t*)(smem + kRingBytes + kRecBytes + 8 * (3 * kSlots + 12));
    uint4* rec_smem = reinterpret_cast<uint4*>(smem + kRingBytes);
    Records rd{rec_smem, bar_rec_full(0), bar_rec_free(0), (int)(threadIdx.x & 31), g.status};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TcStage* table = g.stages + (size_t)blockIdx.x * g.pitch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(bar_full(s), 32 * kLoadWarps);
            mbar_init(bar_conv(s), kConvWarps);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 4; ++a) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_free(a), kEpiWarps);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(bar_rec_full(h), 1);
            mbar_init(bar_rec_free(h), kRoleWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        tmem_alloc(tmem_word, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_word_ptr;

    if (warp < kLoadWarps) {
        // ------------------------------------------------------------ loaders
        int last_dep[4] = {-1, -1, -1, -1};
        // Thread t takes the 16-byte unit j = t & 7 of rows r = t / 8, r + 16, ...: j and the low bits of
        // r, which the swizzles use, are the thread's own.
        const uint32_t t = threadIdx.x, tj = t & 7u, tr = t >> 3;
        const uint32_t a_const = tr * 128u + ((((tj >> 1) ^ tr) & 3u) << 5) + ((tj & 1u) << 4);
        const uint32_t b_const = tr * 128u + (((tj ^ tr) & 7u) << 4);
        for (uint32_t s = 0;; ++s) {
            rd.enter(s);
            const uint4 p0 = rd.part(s, 0);
            const uint32_t flags = p0.z & 0xffu;
            if (flags & kEnd) break;
            const uint4 p1 = rd.part(s, 1), p2 = rd.part(s, 2), p3 = rd.part(s, 3);
            const uint32_t off = (p0.x & 0xffu) << 10, na = (p0.x >> 16) & 0xffu, kt = p0.x >> 24;
            const uint32_t mt = p0.y & 0xffffu, nt = p0.y >> 16, n_mma = p0.z >> 16, kv = (p0.z >> 8) & 0xffu;
            const int dep[4] = {(int)p0.w, (int)p2.w, (int)p3.z, (int)p3.w};
            if (dep[0] > last_dep[0] || dep[1] > last_dep[1] || dep[2] > last_dep[2] || dep[3] > last_dep[3]) {
                if (lane == 0) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (dep[q] > last_dep[q])
                            mbar_wait(bar_empty((uint32_t)dep[q] % kSlots), ((uint32_t)dep[q] / kSlots) & 1, g.status, 0x301);
                }
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 4; ++q) last_dep[q] = max(last_dep[q], dep[q]);
            }
            const float* A = reinterpret_cast<const float*>((uint64_t)p1.x | ((uint64_t)p1.y << 32));
            const float* B = reinterpret_cast<const float*>((uint64_t)p1.z | ((uint64_t)p1.w << 32));
            const size_t a_cs = (size_t)p2.x, b_cs = (size_t)p2.y;
            // A: boxes of [32 k][32 m]; row k is 128 bytes whose 32-byte units are exchanged by k & 3.
            // Only the rows of k-steps that will be issued are written; what lies outside the problem is zero.
            const uint32_t a_dst = ring + off + a_const, k_rows = kt * 8u;
            const float* a_src = A + 4u * tj + (size_t)tr * a_cs;
            for (uint32_t c = 0; c < na; ++c) {
                const uint32_t m = 32u * c + 4u * tj;
                const uint32_t row_bytes = m < mt ? min(16u, (mt - m) * 4u) : 0u;
#pragma unroll
                for (uint32_t i = 0; i < 2; ++i) {
                    const uint32_t k = tr + 16u * i;
                    if (k < k_rows) {
                        const uint32_t bytes = k < kv ? row_bytes : 0u;
                        cp_async_16_zfill(a_dst + c * 4096u + i * 2048u, bytes ? a_src + 32u * c + (size_t)(16u * i) * a_cs : A, bytes);
                    }
                }
            }
            // B: rows of 128 bytes (32 k), their 16-byte units exchanged by n & 7
            const uint32_t b_dst = ring + off + na * 4096u + b_const;
            const uint32_t kb = 4u * tj;
            const uint32_t col_bytes = kb < kv ? min(16u, (kv - kb) * 4u) : 0u;
            const float* b_src = B + kb + (size_t)tr * b_cs;
#pragma unroll 4
            for (uint32_t i = 0; i < 8; ++i) {
                const uint32_t n = tr + 16u * i;
                if (n < n_mma) {
                    const uint32_t bytes = n < nt ? col_bytes : 0u;
                    cp_async_16_zfill(b_dst + i * 2048u, bytes ? b_src + (size_t)(16u * i) * b_cs : B, bytes);
                }
            }
            cp_async_arrive(bar_full(s % kSlots));
        }
    } else if (warp < kConvWarp) {
        // ------------------------------------------------------------ MMA issuers: issuer i has the units u = i mod 4
        // and with them one accumulator; a tcgen05.mma costs its issuing thread 55 - 110 cycles whatever its shape
        const uint32_t me = (uint32_t)(warp - kMmaWarp);
        const uint32_t idesc0 = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | ((uint32_t)(kTile >> 4) << 24);
        const uint64_t da0 = tc_smem_desc(0u, 4096u, 512u, 1u), db0 = tc_smem_desc(0u, 16u, 1024u, 2u);
        uint32_t unit = 0;
        for (uint32_t s = 0;; ++s) {
            rd.enter(s);
            const uint4 p0 = rd.part(s, 0);
            const uint32_t flags = p0.z & 0xffu;
            if (flags & kEnd) break;
            if (lane == 0 && (unit & 3u) == me) {
                const uint32_t off = (p0.x & 0xffu) << 10, raw = ((p0.x >> 8) & 0xffu) << 10, na = (p0.x >> 16) & 0xffu;
                const uint32_t kt = p0.x >> 24, n_mma = p0.z >> 16;
                const uint32_t acc = unit & 3u, use = unit >> 2;
                if ((flags & kFirst) && use > 0) {
                    mbar_wait(bar_acc_free(acc), (use - 1) & 1, g.status, 0x305);
                    tc_fence_after();
                }
                const uint32_t slot = s % kSlots;
                mbar_wait(bar_conv(slot), (s / kSlots) & 1, g.status, 0x302);
                tc_fence_after();
                // M = 128, A MN-major ([32 k][32 m] boxes 4096 bytes apart, swizzle atoms of 4 k-rows 512
                // bytes apart, a k-step of 8 moves 1024 bytes), B K-major (rows of 128 bytes, 8-row
                // atoms 1024 bytes apart, a k-step moves 32 bytes).  Boxes of A beyond `na` are whatever
                // the ring holds there: they only reach accumulator rows that are never stored.
                const uint32_t idesc = idesc0 | ((n_mma >> 3) << 17);
                const uint32_t a_off = (ring + off) >> 4, b_off = a_off + na * 256u, small = raw >> 4;
                uint64_t da_big = da0 + a_off, db_big = db0 + b_off;
                const uint32_t tmem_d = tmem_base + acc * (uint32_t)kTile;
                uint32_t accumulate = (flags & kFirst) ? 0u : 1u;
                for (uint32_t ks = 0; ks < kt; ++ks) {
                    tc_mma_tf32(tmem_d, da_big + small, db_big, idesc, accumulate);
                    tc_mma_tf32(tmem_d, da_big, db_big + small, idesc, 1);
                    tc_mma_tf32(tmem_d, da_big, db_big, idesc, 1);
                    accumulate = 1;
                    da_big += 1024u >> 4;
                    db_big += 32u >> 4;
                }
                tc_commit(bar_empty(slot));  // the stage's bytes are free once these MMAs have read them
                if (flags & kLast) tc_commit(bar_acc_full(acc));
            }
            if (flags & kLast) ++unit;
        }
    } else if (warp < kEpiWarp) {
        // ------------------------------------------------------------ remainders of the raw operands
        const uint32_t t = threadIdx.x - 32u * kConvWarp;
        constexpr uint32_t kStride = 32u * kConvWarps * 16u;  // bytes the converter warps cover together per step
        for (uint32_t s = 0;; ++s) {
            rd.enter(s);
            const uint4 p0 = rd.part(s, 0);
            const uint32_t flags = p0.z & 0xffu;
            if (flags & kEnd) break;
            const uint32_t off = (p0.x & 0xffu) << 10, raw = ((p0.x >> 8) & 0xffu) << 10;
            const uint32_t slot = s % kSlots;
            if (lane == 0) mbar_wait(bar_full(slot), (s / kSlots) & 1, g.status, 0x303);
            __syncwarp();
            const char* big = smem + off;
            char* small = smem + off + raw;
            // raw is a multiple of 2 KB = 128 threads x 16 bytes: every thread has the same trip count
            for (uint32_t c = t * 16u; c < raw; c += 4u * kStride) {
                float4 v[4];
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i)
                    if (c + i * kStride < raw) v[i] = *reinterpret_cast<const float4*>(big + c + i * kStride);
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i)
                    if (c + i * kStride < raw) *reinterpret_cast<float4*>(small + c + i * kStride) = remainder4(v[i]);
            }
            fence_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_conv(slot));
        }
    } else if (warp == kRoleWarps) {
        // ------------------------------------------------------------ record fetcher
        const uint32_t last = (uint32_t)g.pitch - 1;  // records past a CTA's end mark are end marks up to here
        for (uint32_t h = 0;; ++h) {
            uint4 v[2][4];
            bool end = false;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const TcStage* r = table + min(h * 64u + 32u * i + (uint32_t)lane, last);
#pragma unroll
                for (int q = 0; q < 4; ++q) v[i][q] = ld_part(r, q);
                end |= ((v[i][0].z & 0xffffu) & kEnd) != 0;
            }
            if (h >= 2) {
                if (lane == 0) mbar_wait(bar_rec_free(h & 1u), ((h >> 1) - 1) & 1u, g.status, 0x307);
                __syncwarp();
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) rec_smem[(((h & 1u) * 64u) + 32u * i + lane) * 4 + q] = v[i][q];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_rec_full(h & 1u));
            if (__any_sync(0xffffffffu, end)) break;
        }
    } else {
        // ------------------------------------------------------------ epilogue
        // warp w may touch TMEM lanes 32 * (w % 4) .. + 31; lane = row of the unit
        const uint32_t lane_grp = (uint32_t)warp & 3u;
        const uint32_t row = lane_grp * 32u + (uint32_t)lane;
        const bool read_c = g.beta != 0.f;
        uint32_t unit = 0;
        for (uint32_t s = 0;; ++s) {
            rd.enter(s);
            const uint4 p0 = rd.part(s, 0);
            const uint32_t flags = p0.z & 0xffu;
            if (flags & kEnd) break;
            if (flags & kLast) {
                const uint4 p2 = rd.part(s, 2), p3 = rd.part(s, 3);
                const uint32_t mt = p0.y & 0xffffu, nt = p0.y >> 16;
                const size_t c_cs = (size_t)p2.z;
                float* C = reinterpret_cast<float*>((uint64_t)p3.x | ((uint64_t)p3.y << 32)) + row;
                const uint32_t acc = unit & 3u, use = unit >> 2;
                if (lane == 0) mbar_wait(bar_acc_full(acc), use & 1, g.status, 0x304);
                __syncwarp();
                tc_fence_after();
                if (lane_grp * 32u < mt) {
                    const uint32_t taddr = tmem_base + ((lane_grp * 32u) << 16) + acc * (uint32_t)kTile;
                    for (uint32_t c0 = 0; c0 < nt; c0 += 32) {
                        uint32_t r[32];
                        tc_ld32(taddr + c0, r);
                        tc_wait_ld();
                        if (row < mt) {
#pragma unroll
                            for (uint32_t j = 0; j < 32; ++j)
                                if (c0 + j < nt) {
                                    float* p = C + (size_t)(c0 + j) * c_cs;
                                    float v = g.alpha * __uint_as_float(r[j]);
                                    if (read_c) v += g.beta * *p;
                                    *p = v;
                                }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_free(acc));
                ++unit;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

struct UnitRef {
    uint32_t problem;
    int32_t m0, n0;
    int64_t cost;
};

}  // namespace

// Builds the per-CTA stage sequences of a table when every problem
// qualifies for the tcgen05 kernel; otherwise *declined = true and nothing is allocated.
tfb_status grouped_tcgen05_prepare(tfb_ctx* ctx, size_t n, const tfb_gemm_problem* problems, GroupedFast* out,
                                   bool* declined) {
    *declined = true;
    if (n == 0 || env_int("TFB_NO_GROUPED_TCGEN05", 0) || n > (size_t)INT32_MAX) return TFB_OK;
    const int64_t stage_fixed = env_int("TFB_GROUPED_STAGE_COST", 4096);  // a stage's hand-offs, in bytes of memory time
    std::vector<UnitRef> units;
    units.reserve(n);
    for (size_t p = 0; p < n; ++p) {
        const auto& q = problems[p];
        const bool dims_ok = q.m > 0 && q.n > 0 && q.k > 0 && q.k <= kMaxK && q.m < INT32_MAX && q.n < INT32_MAX;
        const bool layout_ok = q.a_rs == 1 && q.b_rs == 1 && q.c_rs == 1 && q.a_cs % 4 == 0 && q.b_cs % 4 == 0 &&
                               q.a_cs >= q.m && q.b_cs >= q.k && q.c_cs >= q.m && q.a_cs < INT32_MAX &&
                               q.b_cs < INT32_MAX && q.c_cs < INT32_MAX;
        const bool align_ok = ((uintptr_t)q.a % 16 == 0) && ((uintptr_t)q.b % 16 == 0) && ((uintptr_t)q.c % 4 == 0);
        if (!dims_ok || !layout_ok || !align_ok) return TFB_OK;
        const int64_t stages = (q.k + kDepth - 1) / kDepth;
        for (int64_t n0 = 0; n0 < q.n; n0 += kTile)
            for (int64_t m0 = 0; m0 < q.m; m0 += kTile) {
                const int64_t mt = std::min<int64_t>(kTile, q.m - m0), nt = std::min<int64_t>(kTile, q.n - n0);
                units.push_back({(uint32_t)p, (int32_t)m0, (int32_t)n0, 4 * (q.k * (mt + nt) + mt * nt) + stages * stage_fixed});
            }
    }
    // Longest units first, each to the CTA with the least work so far.
    std::stable_sort(units.begin(), units.end(), [](const UnitRef& x, const UnitRef& y) { return x.cost > y.cost; });
    const int grid = (int)std::min<size_t>(units.size(), (size_t)ctx->sm_count);
    std::vector<std::vector<uint32_t>> per_cta(grid);
    {
        typedef std::pair<int64_t, int> Load;
        std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
        for (int c = 0; c < grid; ++c) heap.push({0, c});
        for (size_t i = 0; i < units.size(); ++i) {
            Load l = heap.top();
            heap.pop();
            per_cta[l.second].push_back((uint32_t)i);
            heap.push({l.first + units[i].cost, l.second});
        }
    }
    size_t pitch = 0;
    for (const auto& v : per_cta) {
        size_t st = 0;
        for (uint32_t i : v) st += (size_t)((problems[units[i].problem].k + kDepth - 1) / kDepth);
        pitch = std::max(pitch, st);
    }
    pitch += 2;  // the end record, and the record the roles read one ahead
    TcStage end_mark{};
    end_mark.flags = kEnd;
    end_mark.dep0 = end_mark.dep1 = end_mark.dep2 = end_mark.dep3 = -1;
    std::vector<TcStage> table(pitch * (size_t)grid, end_mark);
    struct Live {
        int idx, begin, end;
    };
    for (int c = 0; c < grid; ++c) {
        TcStage* seq = table.data() + (size_t)c * pitch;
        int s = 0, pos = 0, dep = -1, unit_no = 0;
        std::vector<int> newest_of[4];  // newest_of[i][s]: newest stage <= s of a unit of issuer i (-1: none)
        std::deque<Live> live;
        for (uint32_t i : per_cta[c]) {
            const UnitRef& r = units[i];
            const auto& q = problems[r.problem];
            const int mt = (int)std::min<int64_t>(kTile, q.m - r.m0), nt = (int)std::min<int64_t>(kTile, q.n - r.n0);
            const int na = (mt + 31) / 32;
            const int n_mma = (nt + 15) / 16 * 16;
            const int raw = na * 4096 + n_mma * 128;  // a multiple of 2 KB, at most 32 KB
            for (int64_t k0 = 0; k0 < q.k; k0 += kDepth, ++s) {
                // The MMA reads four boxes of A whatever `na` is: keep that reach inside the ring.
                const int need = 2 * raw, reach = std::max(need, raw + 4 * 4096);
                if (pos + reach > kRingBytes) pos = 0;
                int newest = -1;
                for (int j = (int)live.size() - 1; j >= 0; --j)
                    if (live[j].begin < pos + need && pos < live[j].end) {
                        newest = j;
                        break;
                    }
                if (newest >= 0) {
                    dep = live[newest].idx;
                    live.erase(live.begin(), live.begin() + newest + 1);
                }
                dep = std::max(dep, s - kSlots);  // its barrier set is reused
                for (int q = 0; q < 4; ++q) newest_of[q].push_back(q == (unit_no & 3) ? s : (s ? newest_of[q][s - 1] : -1));
                live.push_back({s, pos, pos + need});
                TcStage& st = seq[s];
                st.off_kb = (uint8_t)(pos >> 10);
                st.raw_kb = (uint8_t)(raw >> 10);
                st.na = (uint8_t)na;
                st.kt = (uint8_t)((std::min<int64_t>(kDepth, q.k - k0) + 7) / 8);
                st.mt = (uint16_t)mt;
                st.nt = (uint16_t)nt;
                st.flags = (uint16_t)((k0 == 0 ? kFirst : 0) | (k0 + kDepth >= q.k ? kLast : 0) |
                                      ((int)std::min<int64_t>(kDepth, q.k - k0) << 8));
                st.n_mma = (uint16_t)n_mma;
                st.dep0 = dep >= 0 ? newest_of[0][dep] : -1;
                st.dep1 = dep >= 0 ? newest_of[1][dep] : -1;
                st.dep2 = dep >= 0 ? newest_of[2][dep] : -1;
                st.dep3 = dep >= 0 ? newest_of[3][dep] : -1;
                st.a = (const float*)q.a + r.m0 + k0 * q.a_cs;
                st.b = (const float*)q.b + k0 + (int64_t)r.n0 * q.b_cs;
                st.a_cs = (int32_t)q.a_cs;
                st.b_cs = (int32_t)q.b_cs;
                st.c_cs = (int32_t)q.c_cs;
                st.c = (float*)q.c + r.m0 + (int64_t)r.n0 * q.c_cs;
                pos += need;
            }
            ++unit_no;
        }
    }
    TFB_TRY(out->mem.alloc(ctx, table.size() * sizeof(TcStage)));
    // `table` is pageable: the copy has been staged by the time the call returns.
    TFB_CUDA(cudaMemcpyAsync(out->mem.ptr, table.data(), table.size() * sizeof(TcStage), cudaMemcpyHostToDevice, ctx->stream));
    out->total_units = (int64_t)units.size();
    out->grid = grid;
    out->pitch = (int)pitch;
    out->tcgen05 = true;
    *declined = false;
    return TFB_OK;
}

tfb_status grouped_tcgen05_run(tfb_ctx* ctx, const GroupedFast& f, Scalar alpha, Scalar beta, bool* declined) {
    *declined = true;
    if (alpha.im != 0 || beta.im != 0) return TFB_OK;
    *declined = false;
    GtArgs g;
    g.stages = (const TcStage*)f.mem.ptr;
    g.pitch = f.pitch;
    g.alpha = (float)alpha.re;
    g.beta = (float)beta.re;
    g.status = ctx->dev_status;
    static std::mutex mu;
    static std::map<int, bool> configured;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!configured[ctx->device]) {
            TFB_CUDA(cudaFuncSetAttribute(grouped_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
            configured[ctx->device] = true;
        }
    }
    LaunchScope ls(ctx, "grouped_tcgen05");
    grouped_tc_kernel<<<f.grid, kThreads, kSmemBytes, ctx->stream>>>(g);
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}

}  // namespace tfb
