// Bandwidth-bound strided kernels: permute, element-wise product, reduce, scale.
// They implement `PrimDescriptor::{Permute, ElementwiseMul, Reduce}` and the alpha/beta
// contract of `TensorPrims::execute` (tenferro-prims/src/lib.rs:170-202, 241-244, 300-320)
// on arbitrary signed element strides.
#include "common.h"
#include "scalar_ops.cuh"

namespace tfb {

// ------------------------------------------------------------------ index helpers
__device__ __forceinline__ void divmod(int64_t idx, int64_t e, int64_t& q, int64_t& r) {
    if ((uint64_t)idx <= 0xffffffffull && (uint64_t)e <= 0xffffffffull) {
        uint32_t a = (uint32_t)idx, b = (uint32_t)e;
        uint32_t qq = a / b;
        q = qq;
        r = a - qq * b;
    } else {
        q = idx / e;
        r = idx - q * e;
    }
}

// Decompose a linear index over modes [first, nest.rank) (mode `first` fastest) into offsets.
template <int NT>
__device__ __forceinline__ void decompose(const LoopNest& nest, int first, int64_t idx, int64_t (&off)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) off[t] = 0;
    for (int d = first; d < nest.rank; ++d) {
        int64_t q, r;
        divmod(idx, nest.extent[d], q, r);
#pragma unroll
        for (int t = 0; t < NT; ++t) off[t] += r * nest.stride[t][d];
        idx = q;
    }
}

// ------------------------------------------------------------------ permute
// General path: linear over the nest in OUTPUT order (mode 0 = output's fastest), so writes
// coalesce; reads are whatever the input strides give.
template <typename T>
__global__ void __launch_bounds__(256) permute_generic_kernel(LoopNest nest, const T* __restrict__ in, T* out,
                                                              EpilogueArgs<T> ep) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nest.total; idx += stride) {
        int64_t off[2];
        decompose<2>(nest, 0, idx, off);
        T v = in[off[0]];
        out[off[1]] = ep.apply(v, out + off[1]);
    }
}

// Row path: mode 0 has stride 1 in both tensors.  V elements per thread move as one 16-byte
// access when `vec` holds (alignment checked on the host).
template <typename T, int V>
__global__ void __launch_bounds__(256) permute_rows_kernel(LoopNest nest, const T* __restrict__ in, T* out,
                                                           EpilogueArgs<T> ep) {
    // One "unit" = V consecutive elements of mode 0.
    const int64_t row_units = nest.extent[0] / V;
    const int64_t units = nest.total / V;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (ep.plain) {
        // Pure copy: four units per thread, all loads issued before the first store.
        for (; u + 3 * stride < units; u += 4 * stride) {
            Pack<T, V> p[4];
            T* dst[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int64_t q, r;
                divmod(u + k * stride, row_units, q, r);
                int64_t off[2];
                decompose<2>(nest, 1, q, off);
                p[k] = *reinterpret_cast<const Pack<T, V>*>(in + off[0] + r * V);
                dst[k] = out + off[1] + r * V;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) *reinterpret_cast<Pack<T, V>*>(dst[k]) = p[k];
        }
    }
    for (; u < units; u += stride) {
        int64_t q, r;
        divmod(u, row_units, q, r);
        int64_t off[2];
        decompose<2>(nest, 1, q, off);
        const T* src = in + off[0] + r * V;
        T* dst = out + off[1] + r * V;
        Pack<T, V> p = *reinterpret_cast<const Pack<T, V>*>(src);
        if (ep.plain) {
            *reinterpret_cast<Pack<T, V>*>(dst) = p;
        } else {
            Pack<T, V> o;
            if (ep.read_out) o = *reinterpret_cast<const Pack<T, V>*>(dst);
#pragma unroll
            for (int i = 0; i < V; ++i) o.v[i] = ep.apply(p.v[i], &o.v[i]);
            *reinterpret_cast<Pack<T, V>*>(dst) = o;
        }
    }
}

// Tiled transpose path: mode 0 is the input's stride-1 mode ("i"), mode 1 the output's
// stride-1 mode ("j").  A TILE x TILE patch goes through shared memory so that both the
// reads (along i) and the writes (along j) are full 128-byte lines.
template <typename T>
struct TileOf {
    static constexpr int value = sizeof(T) >= 16 ? 32 : 64;  // keeps the patch under 48 KB
};
template <typename T>
__global__ void __launch_bounds__(256) permute_tiled_kernel(LoopNest nest, const T* __restrict__ in, T* out,
                                                            EpilogueArgs<T> ep, int64_t tiles_i, int64_t tiles_j,
                                                            int64_t n_tiles) {
    constexpr int kTile = TileOf<T>::value;
    constexpr int kStep = 256 / kTile;
    // Odd pitch: a column walk hits distinct banks.
    __shared__ T tile[kTile][kTile + 1];
    const int tx = threadIdx.x % kTile, ty = threadIdx.x / kTile;
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        int64_t q, ti, tj;
        divmod(t, tiles_i, q, ti);
        int64_t rest;
        divmod(q, tiles_j, rest, tj);
        int64_t off[2];
        decompose<2>(nest, 2, rest, off);
        const int64_t i0 = ti * kTile, j0 = tj * kTile;
        const int64_t ni = min((int64_t)kTile, nest.extent[0] - i0), nj = min((int64_t)kTile, nest.extent[1] - j0);
        const T* src = in + off[0] + i0 * nest.stride[0][0] + j0 * nest.stride[0][1];
        T* dst = out + off[1] + i0 * nest.stride[1][0] + j0 * nest.stride[1][1];
        const int64_t s_in_j = nest.stride[0][1], s_out_i = nest.stride[1][0];
        // Load: threads along i (input stride 1).
        if (tx < ni) {
#pragma unroll 4
            for (int j = ty; j < nj; j += kStep) tile[j][tx] = src[tx + j * s_in_j];
        }
        __syncthreads();
        // Store: threads along j (output stride 1).
        if (tx < nj) {
#pragma unroll 4
            for (int i = ty; i < ni; i += kStep) {
                T* p = dst + tx + i * s_out_i;
                *p = ep.apply(tile[tx][i], p);
            }
        }
        __syncthreads();
    }
}

// Vector variant of the tiled transpose for 4- and 8-byte elements: 16-byte loads along the
// input's unit stride, 16-byte stores along the output's, every load of a thread issued before
// the first use (16 KB in flight per CTA; MINB CTAs per SM).  Needs both sides 16-byte aligned.
template <typename T, int V, int MINB>
__global__ void __launch_bounds__(256, MINB) permute_tiled_vec_kernel(LoopNest nest, const T* __restrict__ in, T* out,
                                                                EpilogueArgs<T> ep, int64_t tiles_i, int64_t tiles_j,
                                                                int64_t n_tiles) {
    constexpr int TILE = 64, VPR = TILE / V, LOADS = TILE * TILE / V / 256;
    __shared__ T tile[TILE][TILE + 1];  // tile[i][j]
    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        int64_t q, ti, tj, rest;
        divmod(t, tiles_i, q, ti);
        divmod(q, tiles_j, rest, tj);
        int64_t off[2];
        decompose<2>(nest, 2, rest, off);
        const int64_t i0 = ti * TILE, j0 = tj * TILE;
        const int ni = (int)min((int64_t)TILE, nest.extent[0] - i0), nj = (int)min((int64_t)TILE, nest.extent[1] - j0);
        const T* src = in + off[0] + i0 * nest.stride[0][0] + j0 * nest.stride[0][1];
        T* dst = out + off[1] + i0 * nest.stride[1][0] + j0 * nest.stride[1][1];
        const int64_t s_in_j = nest.stride[0][1], s_out_i = nest.stride[1][0];
        Pack<T, V> v[LOADS];
#pragma unroll
        for (int r = 0; r < LOADS; ++r) {
            const int c = threadIdx.x + 256 * r, i = (c % VPR) * V, j = c / VPR;
            if (i < ni && j < nj) v[r] = *reinterpret_cast<const Pack<T, V>*>(src + i + j * s_in_j);
        }
#pragma unroll
        for (int r = 0; r < LOADS; ++r) {
            const int c = threadIdx.x + 256 * r, i = (c % VPR) * V, j = c / VPR;
            if (i < ni && j < nj) {
#pragma unroll
                for (int e = 0; e < V; ++e) tile[i + e][j] = v[r].v[e];
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < LOADS; ++r) {
            const int c = threadIdx.x + 256 * r, j = (c % VPR) * V, i = c / VPR;
            if (j < nj && i < ni) {
                Pack<T, V>* p = reinterpret_cast<Pack<T, V>*>(dst + j + i * s_out_i);
                Pack<T, V> o;
                if (ep.read_out) o = *p;
#pragma unroll
                for (int e = 0; e < V; ++e) o.v[e] = ep.apply(tile[i][j + e], &o.v[e]);
                *p = o;
            }
        }
        __syncthreads();
    }
}

template <typename T>
static tfb_status permute_typed(tfb_ctx* ctx, const LoopNest& nest_out_order, const void* in, void* out, Scalar alpha,
                                Scalar beta, bool conj) {
    EpilogueArgs<T> ep = EpilogueArgs<T>::make(alpha, beta, conj);
    LoopNest nest = nest_out_order;
    if (nest.total == 0) return TFB_OK;
    const int sms = ctx->sm_count;
    // Row path?
    if (nest.rank >= 1 && nest.stride[0][0] == 1 && nest.stride[1][0] == 1) {
        constexpr int VMAX = 16 / sizeof(T) > 0 ? 16 / sizeof(T) : 1;
        bool vec = VMAX > 1 && nest.extent[0] % VMAX == 0 && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0);
        for (int d = 1; d < nest.rank && vec; ++d)
            vec = nest.stride[0][d] % VMAX == 0 && nest.stride[1][d] % VMAX == 0;
        int64_t units = vec ? nest.total / VMAX : nest.total;
        int64_t blocks = (units + 255) / 256;
        int64_t cap = (int64_t)sms * 16;
        int grid = (int)(blocks < cap ? blocks : cap);
        if (grid < 1) grid = 1;
        LaunchScope ls(ctx, "permute_rows");
        if (vec)
            permute_rows_kernel<T, VMAX><<<grid, 256, 0, ctx->stream>>>(nest, (const T*)in, (T*)out, ep);
        else
            permute_rows_kernel<T, 1><<<grid, 256, 0, ctx->stream>>>(nest, (const T*)in, (T*)out, ep);
        TFB_CUDA(cudaGetLastError());
        return TFB_OK;
    }
    // Tiled transpose?  Find the input's stride-1 mode; it must not be mode 0 (handled above).
    if (nest.rank >= 2 && nest.stride[1][0] == 1) {
        int im = -1;
        for (int d = 1; d < nest.rank; ++d)
            if (nest.stride[0][d] == 1) im = d;
        if (im > 0 && nest.extent[im] >= 16 && nest.extent[0] >= 16) {
            // Reorder: mode 0 <- input-fast mode, mode 1 <- output-fast mode, rest keep order.
            LoopNest r;
            r.rank = nest.rank;
            r.total = nest.total;
            int w = 0;
            auto put = [&](int d) {
                r.extent[w] = nest.extent[d];
                for (int t = 0; t < 3; ++t) r.stride[t][w] = nest.stride[t][d];
                ++w;
            };
            put(im);
            put(0);
            for (int d = 1; d < nest.rank; ++d)
                if (d != im) put(d);
            constexpr int kTile = TileOf<T>::value;
            int64_t ti = (r.extent[0] + kTile - 1) / kTile, tj = (r.extent[1] + kTile - 1) / kTile;
            int64_t rest = 1;
            for (int d = 2; d < r.rank; ++d) rest *= r.extent[d];
            int64_t n_tiles = ti * tj * rest;
            int64_t cap = (int64_t)sms * 32;
            int grid = (int)(n_tiles < cap ? n_tiles : cap);
            LaunchScope ls(ctx, "permute_tiled");
            constexpr int V = 16 / sizeof(T);
            bool vec = V > 1 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0 && r.extent[0] % V == 0 &&
                       r.extent[1] % V == 0;
            for (int d = 0; d < r.rank && vec; ++d) {
                if (d != 0 && r.stride[0][d] % V != 0) vec = false;  // every input stride but the unit one
                if (d != 1 && r.stride[1][d] % V != 0) vec = false;  // every output stride but the unit one
            }
            if constexpr (sizeof(T) <= 8) if (vec) {
                // 64 x 64 tiles whatever the element size
                ti = (r.extent[0] + 63) / 64;
                tj = (r.extent[1] + 63) / 64;
                n_tiles = ti * tj * rest;
                grid = (int)(n_tiles < cap ? n_tiles : cap);
                // CTAs per SM: each holds 16 KB of loads in flight, and HBM wants about 90 KB per SM.
                // Six fit for 4-byte elements (40 registers); the 33 KB tiles of 8-byte elements do
                // best at three.
                constexpr int kOcc = sizeof(T) == 4 ? 6 : 3;
                permute_tiled_vec_kernel<T, (V > 1 ? V : 2), kOcc><<<grid, 256, 0, ctx->stream>>>(r, (const T*)in, (T*)out, ep,
                                                                                                  ti, tj, n_tiles);
                TFB_CUDA(cudaGetLastError());
                return TFB_OK;
            }
            permute_tiled_kernel<T><<<grid, 256, 0, ctx->stream>>>(r, (const T*)in, (T*)out, ep, ti, tj, n_tiles);
            TFB_CUDA(cudaGetLastError());
            return TFB_OK;
        }
    }
    int64_t blocks = (nest.total + 255) / 256;
    int64_t cap = (int64_t)sms * 16;
    int grid = (int)(blocks < cap ? blocks : cap);
    LaunchScope ls(ctx, "permute_generic");
    permute_generic_kernel<T><<<grid, 256, 0, ctx->stream>>>(nest, (const T*)in, (T*)out, ep);
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}

tfb_status launch_permute(tfb_ctx* ctx, int dtype, const LoopNest& nest, const void* in, void* out, Scalar alpha,
                          Scalar beta, bool conj) {
    DeviceGuard g(ctx->device);
    switch (dtype) {
        case TFB_F32: return permute_typed<float>(ctx, nest, in, out, alpha, beta, conj);
        case TFB_F64: return permute_typed<double>(ctx, nest, in, out, alpha, beta, conj);
        case TFB_C32: return permute_typed<float2>(ctx, nest, in, out, alpha, beta, conj);
        case TFB_C64: return permute_typed<double2>(ctx, nest, in, out, alpha, beta, conj);
    }
    return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
}

// ------------------------------------------------------------------ scale (out = beta * out)
template <typename T>
__global__ void __launch_bounds__(256) scale_kernel(LoopNest nest, T* out, T beta, bool zero) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nest.total; idx += stride) {
        int64_t off[1];
        decompose<1>(nest, 0, idx, off);
        out[off[0]] = zero ? Ops<T>::zero() : Ops<T>::mul(beta, out[off[0]]);
    }
}
template <typename T>
static tfb_status scale_typed(tfb_ctx* ctx, const LoopNest& nest, void* out, Scalar beta) {
    if (nest.total == 0 || beta.is_one()) return TFB_OK;
    int64_t blocks = (nest.total + 255) / 256;
    int64_t cap = (int64_t)ctx->sm_count * 16;
    int grid = (int)(blocks < cap ? blocks : cap);
    LaunchScope ls(ctx, "scale");
    scale_kernel<T><<<grid, 256, 0, ctx->stream>>>(nest, (T*)out, Ops<T>::from(beta), beta.is_zero());
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}
tfb_status launch_scale(tfb_ctx* ctx, int dtype, const LoopNest& nest, void* out, Scalar beta) {
    DeviceGuard g(ctx->device);
    switch (dtype) {
        case TFB_F32: return scale_typed<float>(ctx, nest, out, beta);
        case TFB_F64: return scale_typed<double>(ctx, nest, out, beta);
        case TFB_C32: return scale_typed<float2>(ctx, nest, out, beta);
        case TFB_C64: return scale_typed<double2>(ctx, nest, out, beta);
    }
    return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
}

// ------------------------------------------------------------------ element-wise product
template <typename T>
__global__ void __launch_bounds__(256) ewmul_kernel(LoopNest nest, const T* __restrict__ a, const T* __restrict__ b,
                                                    T* out, EpilogueArgs<T> ep, bool conj_a, bool conj_b) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nest.total; idx += stride) {
        int64_t off[3];
        decompose<3>(nest, 0, idx, off);
        T x = a[off[0]], y = b[off[1]];
        if (conj_a) x = Ops<T>::conj(x);
        if (conj_b) y = Ops<T>::conj(y);
        out[off[2]] = ep.apply(Ops<T>::mul(x, y), out + off[2]);
    }
}
template <typename T>
static tfb_status ewmul_typed(tfb_ctx* ctx, const LoopNest& nest, const void* a, const void* b, void* out,
                              Scalar alpha, Scalar beta, bool ca, bool cb) {
    if (nest.total == 0) return TFB_OK;
    EpilogueArgs<T> ep = EpilogueArgs<T>::make(alpha, beta, false);
    int64_t blocks = (nest.total + 255) / 256;
    int64_t cap = (int64_t)ctx->sm_count * 16;
    int grid = (int)(blocks < cap ? blocks : cap);
    LaunchScope ls(ctx, "elementwise_mul");
    ewmul_kernel<T><<<grid, 256, 0, ctx->stream>>>(nest, (const T*)a, (const T*)b, (T*)out, ep, ca, cb);
    TFB_CUDA(cudaGetLastError());
    return TFB_OK;
}
tfb_status launch_elementwise_mul(tfb_ctx* ctx, int dtype, const LoopNest& nest, const void* a, const void* b,
                                  void* out, Scalar alpha, Scalar beta, bool conj_a, bool conj_b) {
    DeviceGuard g(ctx->device);
    switch (dtype) {
        case TFB_F32: return ewmul_typed<float>(ctx, nest, a, b, out, alpha, beta, conj_a, conj_b);
        case TFB_F64: return ewmul_typed<double>(ctx, nest, a, b, out, alpha, beta, conj_a, conj_b);
        case TFB_C32: return ewmul_typed<float2>(ctx, nest, a, b, out, alpha, beta, conj_a, conj_b);
        case TFB_C64: return ewmul_typed<double2>(ctx, nest, a, b, out, alpha, beta, conj_a, conj_b);
    }
    return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
}

// ------------------------------------------------------------------ reduce
// Grid: x over groups of kept elements, y over `splits` slices of the reduced range.
// Two thread layouts:
//   LANES_ON_RED = true : a warp shares one kept element, lanes stride the reduced range
//                         (input stride 1 lies in a reduced mode);
//   LANES_ON_RED = false: each thread owns one kept element and walks its reduced slice
//                         (input stride 1 lies in a kept mode: neighbouring threads coalesce).
// With splits > 1 partial results go to `partial[split][kept]` and reduce_finish_kernel
// combines them in a fixed order, so results do not depend on scheduling.
template <typename T, int OP>
struct Red {
    __device__ static T init() {
        if (OP == TFB_REDUCE_SUM) return Ops<T>::zero();
        if (OP == TFB_REDUCE_MAX) return Ops<T>::lowest();
        return Ops<T>::highest();
    }
    __device__ static T comb(T a, T b) {
        if (OP == TFB_REDUCE_SUM) return Ops<T>::add(a, b);
        if (OP == TFB_REDUCE_MAX) return Ops<T>::max_(a, b);
        return Ops<T>::min_(a, b);
    }
};

template <typename T, int OP, bool LANES_ON_RED>
__global__ void __launch_bounds__(256) reduce_kernel(LoopNest kept, LoopNest red, const T* __restrict__ in, T* out,
                                                     T* partial, int splits, EpilogueArgs<T> ep) {
    const int64_t n_red = red.total;
    const int64_t chunk = (n_red + splits - 1) / splits;
    const int64_t r0 = (int64_t)blockIdx.y * chunk;
    const int64_t r1 = min(n_red, r0 + chunk);
    if (LANES_ON_RED) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int64_t warps_total = (int64_t)gridDim.x * 8;
        for (int64_t ko = (int64_t)blockIdx.x * 8 + warp; ko < kept.total; ko += warps_total) {
            int64_t koff[2];
            decompose<2>(kept, 0, ko, koff);
            // Walk the reduced range in runs along its innermost mode (no division per
            // element); eight independent partial results per lane keep loads in flight.
            T part[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) part[u] = Red<T, OP>::init();
            const int64_t e0 = red.extent[0], s0 = red.stride[0][0];
            int64_t r = r0;
            while (r < r1) {
                int64_t q, i0;
                divmod(r, e0, q, i0);
                int64_t roff[1];
                decompose<1>(red, 1, q, roff);
                const int64_t run = min(e0 - i0, r1 - r);
                const T* p = in + koff[0] + roff[0] + i0 * s0;
                int64_t i = lane;
                for (; i + 224 < run; i += 256) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) part[u] = Red<T, OP>::comb(part[u], p[(i + 32 * u) * s0]);
                }
                for (; i < run; i += 32) part[0] = Red<T, OP>::comb(part[0], p[i * s0]);
                r += run;
            }
            T acc = Red<T, OP>::comb(Red<T, OP>::comb(Red<T, OP>::comb(part[0], part[1]), Red<T, OP>::comb(part[2], part[3])),
                                     Red<T, OP>::comb(Red<T, OP>::comb(part[4], part[5]), Red<T, OP>::comb(part[6], part[7])));
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) acc = Red<T, OP>::comb(acc, Ops<T>::shfl_down(acc, s));
            if (lane == 0) {
                if (splits == 1)
                    out[koff[1]] = ep.apply(acc, out + koff[1]);
                else
                    partial[(int64_t)blockIdx.y * kept.total + ko] = acc;
            }
        }
    } else {
        const int64_t threads_total = (int64_t)gridDim.x * blockDim.x;
        for (int64_t ko = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ko < kept.total; ko += threads_total) {
            int64_t koff[2];
            decompose<2>(kept, 0, ko, koff);
            T acc = Red<T, OP>::init();
            // Walk the reduced range mode 0 innermost without re-dividing per element.
            const int64_t e0 = red.extent[0], s0 = red.stride[0][0];
            int64_t r = r0;
            while (r < r1) {
                int64_t q, i0;
                divmod(r, e0, q, i0);
                int64_t roff[1];
                decompose<1>(red, 1, q, roff);
                int64_t run = min(e0 - i0, r1 - r);
                const T* p = in + koff[0] + roff[0] + i0 * s0;
                for (int64_t i = 0; i < run; ++i) acc = Red<T, OP>::comb(acc, p[i * s0]);
                r += run;
            }
            if (splits == 1)
                out[koff[1]] = ep.apply(acc, out + koff[1]);
            else
                partial[(int64_t)blockIdx.y * kept.total + ko] = acc;
        }
    }
}

template <typename T, int OP>
__global__ void __launch_bounds__(256) reduce_finish_kernel(LoopNest kept, const T* __restrict__ partial, T* out,
                                                            int splits, EpilogueArgs<T> ep) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t ko = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ko < kept.total; ko += stride) {
        int64_t koff[2];
        decompose<2>(kept, 0, ko, koff);
        T acc = partial[ko];
        for (int s = 1; s < splits; ++s) acc = Red<T, OP>::comb(acc, partial[(int64_t)s * kept.total + ko]);
        out[koff[1]] = ep.apply(acc, out + koff[1]);
    }
}

template <typename T, int OP>
static tfb_status reduce_typed(tfb_ctx* ctx, const LoopNest& kept, const LoopNest& red, const void* in, void* out,
                               Scalar alpha, Scalar beta, bool conj) {
    if (kept.total == 0) return TFB_OK;
    EpilogueArgs<T> ep = EpilogueArgs<T>::make(alpha, beta, conj);
    if (red.total == 0) {
        // Empty reduction: Sum gives 0; Max/Min over nothing is rejected at plan time.
        return launch_scale(ctx, std::is_same<T, float>::value    ? TFB_F32
                                 : std::is_same<T, double>::value ? TFB_F64
                                 : std::is_same<T, float2>::value ? TFB_C32
                                                                  : TFB_C64,
                            [&] {
                                LoopNest o = kept;
                                for (int d = 0; d < o.rank; ++d) o.stride[0][d] = kept.stride[1][d];
                                return o;
                            }(),
                            out, beta);
    }
    // Which layout?  Smallest |input stride| among reduced vs kept modes.
    auto min_stride = [](const LoopNest& n) {
        int64_t m = INT64_MAX;
        for (int d = 0; d < n.rank; ++d) {
            int64_t s = n.stride[0][d] < 0 ? -n.stride[0][d] : n.stride[0][d];
            if (n.extent[d] > 1 && s < m) m = s;
        }
        return m;
    };
    const bool lanes_on_red = kept.rank == 0 || min_stride(red) < min_stride(kept);
    const int sms = ctx->sm_count;
    int64_t groups = lanes_on_red ? (kept.total + 7) / 8 : (kept.total + 255) / 256;
    int64_t target = (int64_t)sms * 8;
    int splits = 1;
    if (groups < target) {
        int64_t want = target / (groups > 0 ? groups : 1);
        int64_t min_chunk = lanes_on_red ? 1024 : 64;
        int64_t max_splits = (red.total + min_chunk - 1) / min_chunk;
        splits = (int)(want < max_splits ? want : max_splits);
        if (splits < 1) splits = 1;
        if (splits > 1024) splits = 1024;
    }
    int64_t gx = groups < target * 4 ? groups : target * 4;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)splits);
    PoolBlock ws;
    T* partial = nullptr;
    if (splits > 1) {
        TFB_TRY(ws.alloc(ctx, sizeof(T) * (size_t)splits * (size_t)kept.total));
        partial = (T*)ws.ptr;
    }
    {
    LaunchScope ls(ctx, "reduce");
    if (lanes_on_red)
        reduce_kernel<T, OP, true><<<grid, 256, 0, ctx->stream>>>(kept, red, (const T*)in, (T*)out, partial, splits, ep);
    else
        reduce_kernel<T, OP, false><<<grid, 256, 0, ctx->stream>>>(kept, red, (const T*)in, (T*)out, partial, splits,
                                                                   ep);
    }
    TFB_CUDA(cudaGetLastError());
    if (splits > 1) {
        int64_t blocks = (kept.total + 255) / 256;
        int g2 = (int)(blocks < (int64_t)sms * 8 ? blocks : (int64_t)sms * 8);
        LaunchScope ls(ctx, "reduce_finish");
        reduce_finish_kernel<T, OP><<<g2, 256, 0, ctx->stream>>>(kept, partial, (T*)out, splits, ep);
        TFB_CUDA(cudaGetLastError());
    }
    return TFB_OK;
}

template <typename T>
static tfb_status reduce_op_dispatch(tfb_ctx* ctx, int op, const LoopNest& kept, const LoopNest& red, const void* in,
                                     void* out, Scalar alpha, Scalar beta, bool conj) {
    switch (op) {
        case TFB_REDUCE_SUM: return reduce_typed<T, TFB_REDUCE_SUM>(ctx, kept, red, in, out, alpha, beta, conj);
        case TFB_REDUCE_MAX: return reduce_typed<T, TFB_REDUCE_MAX>(ctx, kept, red, in, out, alpha, beta, conj);
        case TFB_REDUCE_MIN: return reduce_typed<T, TFB_REDUCE_MIN>(ctx, kept, red, in, out, alpha, beta, conj);
    }
    return fail(TFB_ERR_INVALID_ARGUMENT, "unknown reduce op %d", op);
}

tfb_status launch_reduce(tfb_ctx* ctx, int dtype, int op, const LoopNest& kept, const LoopNest& red, const void* in,
                         void* out, Scalar alpha, Scalar beta, bool conj) {
    DeviceGuard g(ctx->device);
    switch (dtype) {
        case TFB_F32: return reduce_op_dispatch<float>(ctx, op, kept, red, in, out, alpha, beta, conj);
        case TFB_F64: return reduce_op_dispatch<double>(ctx, op, kept, red, in, out, alpha, beta, conj);
        case TFB_C32:
            if (op != TFB_REDUCE_SUM) return fail(TFB_ERR_INVALID_ARGUMENT, "Max/Min are undefined for complex types");
            return reduce_typed<float2, TFB_REDUCE_SUM>(ctx, kept, red, in, out, alpha, beta, conj);
        case TFB_C64:
            if (op != TFB_REDUCE_SUM) return fail(TFB_ERR_INVALID_ARGUMENT, "Max/Min are undefined for complex types");
            return reduce_typed<double2, TFB_REDUCE_SUM>(ctx, kept, red, in, out, alpha, beta, conj);
    }
    return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
}

// ------------------------------------------------------------------ reduce without allocation
// Some callers must not allocate device memory when they call in: an application that has
// handed all device memory to an allocator of its own, a latency-critical loop that cannot
// afford the pool's occasional trip to the driver, a framework callback in which device
// allocation is forbidden.  For them the split partials of the reduce kernel live in this
// fixed array instead of a pool block.  Every GPU that loads the library carries these
// 4 MiB until the process exits.
constexpr size_t kStaticReduceBytes = (size_t)4 << 20;
static __device__ __align__(256) unsigned char g_static_reduce_scratch[kStaticReduceBytes];

// In host code the array's name is only a handle for the runtime, not an address a kernel
// could use: the device address is asked for once per device, with that device current.
static tfb_status static_reduce_scratch(tfb_ctx* ctx, void** out) {
    static std::mutex mu;
    static std::map<int, void*> by_device;
    std::lock_guard<std::mutex> lock(mu);
    auto it = by_device.find(ctx->device);
    if (it != by_device.end()) {
        *out = it->second;
        return TFB_OK;
    }
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_reduce_scratch);
    if (e != cudaSuccess || !ptr)
        return fail(TFB_ERR_DEVICE, "cudaGetSymbolAddress(static reduce scratch) failed on device %d: %s", ctx->device,
                    cudaGetErrorString(e));
    by_device[ctx->device] = ptr;
    *out = ptr;
    return TFB_OK;
}

template <typename T, int OP>
static tfb_status reduce_static_typed(tfb_ctx* ctx, const LoopNest& kept, const LoopNest& red, const void* in, void* out,
                                      Scalar alpha, Scalar beta, bool conj, void* scratch) {
    EpilogueArgs<T> ep = EpilogueArgs<T>::make(alpha, beta, conj);
    auto min_stride = [](const LoopNest& n) {
        int64_t m = INT64_MAX;
        for (int d = 0; d < n.rank; ++d) {
            int64_t s = n.stride[0][d] < 0 ? -n.stride[0][d] : n.stride[0][d];
            if (n.extent[d] > 1 && s < m) m = s;
        }
        return m;
    };
    const bool lanes_on_red = kept.rank == 0 || min_stride(red) < min_stride(kept);
    const int sms = ctx->sm_count;
    const int64_t groups = lanes_on_red ? (kept.total + 7) / 8 : (kept.total + 255) / 256;
    const int64_t target = (int64_t)sms * 8;
    int64_t splits = 1;
    if (groups < target) {
        const int64_t want = target / (groups > 0 ? groups : 1);
        const int64_t min_chunk = lanes_on_red ? 1024 : 64;
        const int64_t max_splits = (red.total + min_chunk - 1) / min_chunk;
        splits = want < max_splits ? want : max_splits;
        // The partials have to fit the fixed array.
        const int64_t fit = (int64_t)(kStaticReduceBytes / (sizeof(T) * (size_t)kept.total));
        if (splits > fit) splits = fit;
        if (splits > 1024) splits = 1024;
        if (splits < 1) splits = 1;
    }
    int64_t gx = groups < target * 4 ? groups : target * 4;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)splits);
    T* partial = splits > 1 ? (T*)scratch : nullptr;
    count_launch(1);
    if (lanes_on_red)
        reduce_kernel<T, OP, true><<<grid, 256, 0, ctx->stream>>>(kept, red, (const T*)in, (T*)out, partial, (int)splits, ep);
    else
        reduce_kernel<T, OP, false><<<grid, 256, 0, ctx->stream>>>(kept, red, (const T*)in, (T*)out, partial, (int)splits,
                                                                   ep);
    TFB_CUDA(cudaGetLastError());
    if (splits > 1) {
        const int64_t blocks = (kept.total + 255) / 256;
        const int g2 = (int)(blocks < (int64_t)sms * 8 ? blocks : (int64_t)sms * 8);
        count_launch(1);
        reduce_finish_kernel<T, OP><<<g2, 256, 0, ctx->stream>>>(kept, partial, (T*)out, (int)splits, ep);
        TFB_CUDA(cudaGetLastError());
    }
    return TFB_OK;
}

template <typename T>
static tfb_status reduce_static_ops(tfb_ctx* ctx, int op, const LoopNest& kept, const LoopNest& red, const void* in,
                                    void* out, Scalar alpha, Scalar beta, bool conj, void* scratch) {
    switch (op) {
        case TFB_REDUCE_SUM: return reduce_static_typed<T, TFB_REDUCE_SUM>(ctx, kept, red, in, out, alpha, beta, conj, scratch);
        case TFB_REDUCE_MAX: return reduce_static_typed<T, TFB_REDUCE_MAX>(ctx, kept, red, in, out, alpha, beta, conj, scratch);
        case TFB_REDUCE_MIN: return reduce_static_typed<T, TFB_REDUCE_MIN>(ctx, kept, red, in, out, alpha, beta, conj, scratch);
    }
    return fail(TFB_ERR_INVALID_ARGUMENT, "unknown reduce op %d", op);
}

}  // namespace tfb

// See include/tenferro_b200.h.  The first call on a device looks up the scratch address
// (cudaGetSymbolAddress); after that a call is two kernel launches and nothing else.
extern "C" tfb_status tfb_reduce_static(tfb_ctx* ctx, int32_t dtype, int32_t reduce_op, const uint32_t* modes_a,
                                        size_t n_modes_a, const tfb_view* a, const uint32_t* modes_c, size_t n_modes_c,
                                        const tfb_view* c, const void* alpha, const void* beta) {
    using namespace tfb;
    if (!ctx || !a || !c || !alpha || !beta) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_reduce_static: NULL argument");
    if (!dtype_valid(dtype)) return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", (int)dtype);
    if (reduce_op < TFB_REDUCE_SUM || reduce_op > TFB_REDUCE_MIN)
        return fail(TFB_ERR_INVALID_ARGUMENT, "unknown reduce op %d", (int)reduce_op);
    if (reduce_op != TFB_REDUCE_SUM && dtype_is_complex(dtype))
        return fail(TFB_ERR_INVALID_ARGUMENT, "Max/Min are undefined for complex types");
    if (a->rank != n_modes_a) return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (input)", n_modes_a, a->rank);
    if (c->rank != n_modes_c) return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (output)", n_modes_c, c->rank);
    if ((n_modes_a && !modes_a) || (n_modes_c && !modes_c)) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_reduce_static: modes are NULL");
    HView va, vc;
    TFB_TRY(to_hview(*a, dtype, &va, "input"));
    TFB_TRY(to_hview(*c, dtype, &vc, "output"));
    if (vc.conj) return fail(TFB_ERR_INVALID_ARGUMENT, "the output view cannot carry the conjugate flag");
    for (size_t i = 0; i < n_modes_a; ++i)
        for (size_t j = i + 1; j < n_modes_a; ++j)
            if (modes_a[i] == modes_a[j]) return fail(TFB_ERR_INVALID_ARGUMENT, "modes_a holds a repeated label");
    std::vector<Mode> kept, red;
    std::vector<bool> used(n_modes_a, false);
    for (size_t i = 0; i < n_modes_c; ++i) {
        size_t j = 0;
        while (j < n_modes_a && modes_a[j] != modes_c[i]) ++j;
        if (j == n_modes_a || used[j]) return fail(TFB_ERR_INVALID_ARGUMENT, "modes_c is not a subset of modes_a (label %u)", modes_c[i]);
        if (va.dims[j] != vc.dims[i])
            return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (label %u)", (long long)va.dims[j],
                        (long long)vc.dims[i], modes_c[i]);
        used[j] = true;
        kept.push_back(Mode{va.dims[j], {va.strides[j], vc.strides[i], 0}});
    }
    for (size_t j = 0; j < n_modes_a; ++j)
        if (!used[j]) red.push_back(Mode{va.dims[j], {va.strides[j], 0, 0}});
    int64_t kept_total = 1, red_total = 1;
    for (auto& m : kept) kept_total *= m.extent;
    for (auto& m : red) red_total *= m.extent;
    if (kept_total == 0) return TFB_OK;
    if (red_total == 0) {
        // As a Reduce plan does: the sum over nothing is 0, so C = beta * C (one launch, no
        // scratch); Max/Min over nothing have no value.
        if (reduce_op != TFB_REDUCE_SUM)
            return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_reduce_static: Max/Min over an empty range is undefined");
        sort_and_fuse(kept, 1, 2);
        for (auto& m : kept) m.s[0] = m.s[1];
        LoopNest nk0;
        TFB_TRY(make_nest(kept, &nk0));
        DeviceGuard guard0(ctx->device);
        return launch_scale(ctx, dtype, nk0, vc.ptr, load_scalar(dtype, beta));
    }
    const size_t out_bytes = (size_t)kept_total * dtype_size(dtype);
    if (out_bytes > kStaticReduceBytes / 2)
        return fail(TFB_ERR_INVALID_ARGUMENT,
                    "tfb_reduce_static: the output holds %zu bytes, more than the %zu this allocation-free entry point "
                    "supports; use tfb_execute with a Reduce plan",
                    out_bytes, kStaticReduceBytes / 2);
    sort_and_fuse(kept, 1, 2);
    sort_and_fuse(red, 0, 1);
    LoopNest nk, nr;
    TFB_TRY(make_nest(kept, &nk));
    TFB_TRY(make_nest(red, &nr));
    DeviceGuard guard(ctx->device);
    void* scratch = nullptr;
    TFB_TRY(static_reduce_scratch(ctx, &scratch));
    const Scalar al = load_scalar(dtype, alpha), be = load_scalar(dtype, beta);
    switch (dtype) {
        case TFB_F32: return reduce_static_ops<float>(ctx, reduce_op, nk, nr, va.ptr, vc.ptr, al, be, va.conj, scratch);
        case TFB_F64: return reduce_static_ops<double>(ctx, reduce_op, nk, nr, va.ptr, vc.ptr, al, be, va.conj, scratch);
        case TFB_C32:
            return reduce_static_typed<float2, TFB_REDUCE_SUM>(ctx, nk, nr, va.ptr, vc.ptr, al, be, va.conj, scratch);
        case TFB_C64:
            return reduce_static_typed<double2, TFB_REDUCE_SUM>(ctx, nk, nr, va.ptr, vc.ptr, al, be, va.conj, scratch);
    }
    return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", (int)dtype);
}
