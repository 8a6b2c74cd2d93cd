// Shared device-side pieces of the contraction kernels: the argument block, the offset
// ("scatter") tables that carry arbitrary strides into the GEMM main loop, and the
// cp.async helpers.
//
// A contraction `C[modes_c] = alpha * A[modes_a] . B[modes_b] + beta * C`
// (tenferro-prims/src/lib.rs:227-239) is normalised on the host into four mode groups:
// batch (in A, B and C), M (A and C), N (B and C), K (A and B).  Each group is linearised,
// and for every linear index the element offset it contributes in each tensor is tabulated
// once:   addr(A[b,m,k]) = a + a_b[b] + a_m[m] + a_k[k]   and likewise for B and C.
// That is the whole "permute" of permute-into-GEMM: tiles are gathered straight from the
// strided operands, nothing is packed in global memory.
#pragma once
#include "common.h"

namespace tfb {

struct ContractArgs {
    const char* a;
    const char* b;
    char* c;
    const int64_t* a_b;
    const int64_t* b_b;
    const int64_t* c_b;
    const int64_t* a_m;
    const int64_t* c_m;
    const int64_t* b_n;
    const int64_t* c_n;
    const int64_t* a_k;
    const int64_t* b_k;
    int64_t M, N, K, B;
    double alpha_re, alpha_im, beta_re, beta_im;
    int conj_a, conj_b;
    // Fused trailing multiplier D[b,m,n] (nullptr: none): C = alpha * (A B) . D + beta * C.
    const char* mul;
    const int64_t* d_b;
    const int64_t* d_m;
    const int64_t* d_n;
    int conj_mul;
    int a_kfast, b_kfast;  // 1: the unit-stride direction of the operand tile is K; 0: M (resp. N)
    int a_vec, b_vec;      // elements per cp.async (1, or 2 for f64 when 16-byte chunks are legal)
    // Work decomposition: tiles x k-iterations, cut into equal contiguous ranges ("stream-K").
    int64_t tiles_m, tiles_n, n_tiles, k_iters, total_iters, iters_per_cta;
    unsigned* sk_flags;  // per-CTA flags of the in-kernel stream-K reduction (TMA-fed DMMA kernel)
    unsigned sk_epoch;   // a flag is raised when it equals this launch's epoch
    int sk_two_phase;    // 1: every range parks its sums in its slot; a finishing kernel adds the pieces of a tile
    char* partial;  // 2 slots of one block tile per CTA, used only by ranges that cut a tile
};

// The fused multiplier's element at offset `off` (in elements), applied to a real or complex sum.
__device__ __forceinline__ void apply_mul_f64(const ContractArgs& g, int64_t off, double& x) {
    x *= *reinterpret_cast<const double*>(g.mul + off * 8);
}
__device__ __forceinline__ void apply_mul_c128(const ContractArgs& g, int64_t off, double& xr, double& xi) {
    const double2 d = *reinterpret_cast<const double2*>(g.mul + off * 16);
    const double di = g.conj_mul ? -d.y : d.y;
    const double r = xr * d.x - xi * di;
    xi = xr * di + xi * d.x;
    xr = r;
}

// Multiplies a thread's m16n8 accumulator fragments (TM x TN of them, element (i, j, e) at row
// m_first + 8 i, column n_first + 8 j + e; complex sums keep the imaginary part at [2 + e]) by the
// fused multiplier, before anything is stored: with no store in between, all the loads are in flight
// together.  A load placed after a store through an unrelated pointer would wait for that store.
template <bool CPLX, int TM, int TN, int W>
__device__ __forceinline__ void apply_mul_fragments(const ContractArgs& g, int64_t bb, int64_t m_first, int64_t n_first,
                                                    double (&acc)[TM][TN][W]) {
    const int64_t db = g.d_b[bb];
#pragma unroll
    for (int j = 0; j < TN; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int64_t n = n_first + 8 * j + e;
            if (n >= g.N) continue;
            const int64_t dn = db + g.d_n[n];
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const int64_t m = m_first + 8 * i;
                if (m >= g.M) continue;
                if constexpr (CPLX) apply_mul_c128(g, dn + g.d_m[m], acc[i][j][e], acc[i][j][2 + e]);
                else apply_mul_f64(g, dn + g.d_m[m], acc[i][j][e]);
            }
        }
    }
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_8(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int sz = valid ? 8 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int sz = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

}  // namespace tfb
