// TensorPrims<Standard> for the CUDA backend: descriptor validation (plan) and dispatch
// (execute).  Reference protocol: tenferro-prims/src/lib.rs:152-245 (PrimDescriptor),
// :278-340 (TensorPrims::{plan, execute, has_extension_for}).
//
// Every descriptor is lowered to one of two label forms:
//   unary   out[labels_out] = alpha * reduce(in[labels_in]) + beta * out
//   binary  C[labels_c]     = alpha * sum A[labels_a] * B[labels_b] + beta * C
// A label repeated inside one tensor addresses that tensor's diagonal (its strides add up),
// which is how Trace / AntiTrace / AntiDiag and einsum forms like "ii->i", "i->ii" run
// without dedicated kernels.
#include "prims.h"

#include <algorithm>
#include <set>

namespace tfb {

// ------------------------------------------------------------------ mode lists
void fuse_in_order(std::vector<Mode>& modes, int n_tensors) {
    std::vector<Mode> out;
    for (auto& m : modes) {
        if (m.extent == 1) continue;
        if (!out.empty()) {
            Mode& p = out.back();
            bool ok = true;
            for (int t = 0; t < n_tensors; ++t)
                if (m.s[t] != p.s[t] * p.extent) ok = false;
            if (ok) {
                p.extent *= m.extent;
                continue;
            }
        }
        out.push_back(m);
    }
    modes.swap(out);
}

void sort_and_fuse(std::vector<Mode>& modes, int key, int n_tensors) {
    auto mag = [](int64_t v) { return v < 0 ? -v : v; };
    std::stable_sort(modes.begin(), modes.end(), [&](const Mode& x, const Mode& y) {
        // Stride 0 (broadcast) sorts last: it says nothing about locality.
        int64_t a = mag(x.s[key]), b = mag(y.s[key]);
        if ((a == 0) != (b == 0)) return b == 0;
        return a < b;
    });
    fuse_in_order(modes, n_tensors);
}

tfb_status make_nest(const std::vector<Mode>& modes, LoopNest* out) {
    if ((int)modes.size() > kMaxRank)
        return fail(TFB_ERR_INVALID_ARGUMENT, "more than %d non-fusable modes in one operation", kMaxRank);
    out->rank = (int)modes.size();
    out->total = 1;
    for (int d = 0; d < kMaxRank; ++d) {
        out->extent[d] = 1;
        for (int t = 0; t < 3; ++t) out->stride[t][d] = 0;
    }
    for (int d = 0; d < out->rank; ++d) {
        out->extent[d] = modes[d].extent;
        for (int t = 0; t < 3; ++t) out->stride[t][d] = modes[d].s[t];
        out->total *= modes[d].extent;
    }
    return TFB_OK;
}

tfb_status to_hview(const tfb_view& v, int dtype, HView* out, const char* what) {
    if (v.rank > 0 && (!v.dims || !v.strides)) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: dims/strides are NULL", what);
    out->dims.assign(v.rank, 0);
    out->strides.assign(v.rank, 0);
    int64_t n = 1;
    for (size_t i = 0; i < v.rank; ++i) {
        out->dims[i] = (int64_t)v.dims[i];
        out->strides[i] = (int64_t)v.strides[i];
        n *= out->dims[i];
    }
    if (n > 0 && !v.base) return fail(TFB_ERR_INVALID_ARGUMENT, "%s: base pointer is NULL", what);
    out->ptr = (char*)v.base + (int64_t)v.offset * (int64_t)dtype_size(dtype);
    out->conj = (v.flags & TFB_VIEW_CONJ) != 0 && dtype_is_complex(dtype);
    return TFB_OK;
}

// Labelled tensor: unique labels with extent and stride (repeats already merged).
struct Labelled {
    std::vector<uint32_t> labels;
    std::vector<int64_t> extent, stride;
    int find(uint32_t l) const {
        for (size_t i = 0; i < labels.size(); ++i)
            if (labels[i] == l) return (int)i;
        return -1;
    }
};

// Merge repeated labels (diagonal: strides add).  `had_repeats` reports whether any merged.
static tfb_status merge_repeats(const std::vector<uint32_t>& labels, const HView& v, Labelled* out, bool* had_repeats,
                                const char* what) {
    if (labels.size() != v.dims.size())
        return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (%s)", labels.size(), v.dims.size(),
                    what);
    *had_repeats = false;
    for (size_t i = 0; i < labels.size(); ++i) {
        int j = out->find(labels[i]);
        if (j < 0) {
            out->labels.push_back(labels[i]);
            out->extent.push_back(v.dims[i]);
            out->stride.push_back(v.strides[i]);
        } else {
            if (out->extent[j] != v.dims[i])
                return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (repeated label %u in %s)",
                            (long long)out->extent[j], (long long)v.dims[i], labels[i], what);
            out->stride[j] += v.strides[i];
            *had_repeats = true;
        }
    }
    return TFB_OK;
}

static tfb_status full_nest_of(const HView& v, LoopNest* nest) {
    std::vector<Mode> modes;
    for (size_t i = 0; i < v.dims.size(); ++i) modes.push_back(Mode{v.dims[i], {v.strides[i], 0, 0}});
    sort_and_fuse(modes, 0, 1);
    return make_nest(modes, nest);
}

// ------------------------------------------------------------------ unary
tfb_status run_unary(tfb_ctx* ctx, int dtype, const std::vector<uint32_t>& labels_in, const HView& in,
                     const std::vector<uint32_t>& labels_out, const HView& out, Scalar alpha, Scalar beta,
                     int reduce_op, const char** used) {
    Labelled li, lo;
    bool rep_in = false, rep_out = false;
    TFB_TRY(merge_repeats(labels_in, in, &li, &rep_in, "input"));
    TFB_TRY(merge_repeats(labels_out, out, &lo, &rep_out, "output"));
    if (out.conj) return fail(TFB_ERR_INVALID_ARGUMENT, "the output view cannot carry the conjugate flag");
    // Extents of shared labels must agree.
    for (size_t i = 0; i < lo.labels.size(); ++i) {
        int j = li.find(lo.labels[i]);
        if (j >= 0 && li.extent[j] != lo.extent[i])
            return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (label %u)",
                        (long long)li.extent[j], (long long)lo.extent[i], lo.labels[i]);
    }
    if (rep_out) {
        // Only the diagonal receives alpha * in; everything else is beta * out.
        LoopNest all;
        TFB_TRY(full_nest_of(out, &all));
        TFB_TRY(launch_scale(ctx, dtype, all, out.ptr, beta));
        if (!beta.is_zero()) beta = Scalar{1.0, 0.0};
    }
    std::vector<Mode> kept, red;
    for (size_t i = 0; i < lo.labels.size(); ++i) {
        int j = li.find(lo.labels[i]);
        kept.push_back(Mode{lo.extent[i], {j >= 0 ? li.stride[j] : 0, lo.stride[i], 0}});
    }
    for (size_t j = 0; j < li.labels.size(); ++j)
        if (lo.find(li.labels[j]) < 0) red.push_back(Mode{li.extent[j], {li.stride[j], 0, 0}});
    int64_t red_total = 1;
    for (auto& m : red) red_total *= m.extent;
    if (red.empty() || (red_total == 1)) {
        // Pure data movement (the reduced labels, if any, all have extent 1).
        sort_and_fuse(kept, 1, 2);
        LoopNest nest;
        TFB_TRY(make_nest(kept, &nest));
        if (used) *used = "permute";
        return launch_permute(ctx, dtype, nest, in.ptr, out.ptr, alpha, beta, in.conj);
    }
    if (reduce_op != TFB_REDUCE_SUM && red_total == 0)
        return fail(TFB_ERR_INVALID_ARGUMENT, "Max/Min over an empty range is undefined");
    sort_and_fuse(kept, 1, 2);
    sort_and_fuse(red, 0, 1);
    LoopNest nk, nr;
    TFB_TRY(make_nest(kept, &nk));
    TFB_TRY(make_nest(red, &nr));
    if (used) *used = "reduce";
    return launch_reduce(ctx, dtype, reduce_op, nk, nr, in.ptr, out.ptr, alpha, beta, in.conj);
}

// ------------------------------------------------------------------ binary
tfb_status run_binary(tfb_ctx* ctx, int dtype, const std::vector<uint32_t>& labels_a, const HView& a,
                      const std::vector<uint32_t>& labels_b, const HView& b, const std::vector<uint32_t>& labels_c,
                      const HView& c, Scalar alpha, Scalar beta, int force_kernel, const char** used,
                      const std::vector<uint32_t>* labels_d, const HView* d, int algebra) {
    Labelled la, lb, lc, ld;
    bool ra = false, rb = false, rc = false, rd = false;
    TFB_TRY(merge_repeats(labels_a, a, &la, &ra, "first input"));
    TFB_TRY(merge_repeats(labels_b, b, &lb, &rb, "second input"));
    TFB_TRY(merge_repeats(labels_c, c, &lc, &rc, "output"));
    if (d) {
        TFB_TRY(merge_repeats(*labels_d, *d, &ld, &rd, "multiplier"));
        for (auto l : ld.labels)
            if (lc.find(l) < 0 || rc)
                return fail(TFB_ERR_INVALID_ARGUMENT, "a fused multiplier may only carry labels of a plain output");
    }
    if (c.conj) return fail(TFB_ERR_INVALID_ARGUMENT, "the output view cannot carry the conjugate flag");
    if (algebra != TFB_ALGEBRA_STANDARD && (rc || d))
        return fail(TFB_ERR_INVALID_ARGUMENT,
                    "repeated output labels (AntiTrace, AntiDiag) and fused multipliers are implemented for the Standard "
                    "algebra only");
    if (rc) {
        LoopNest all;
        TFB_TRY(full_nest_of(c, &all));
        TFB_TRY(launch_scale(ctx, dtype, all, c.ptr, beta));
        if (!beta.is_zero()) beta = Scalar{1.0, 0.0};
    }
    ContractProblem p;
    p.dtype = dtype;
    p.a = a.ptr;
    p.b = b.ptr;
    p.c = c.ptr;
    p.conj_a = a.conj;
    p.conj_b = b.conj;
    p.alpha = alpha;
    p.beta = beta;
    if (d) {
        p.mul = d->ptr;
        p.conj_mul = d->conj;
    }
    std::set<uint32_t> seen;
    auto classify = [&](uint32_t l) -> tfb_status {
        if (!seen.insert(l).second) return TFB_OK;
        int ia = la.find(l), ib = lb.find(l), ic = lc.find(l), id = d ? ld.find(l) : -1;
        int64_t e = ia >= 0 ? la.extent[ia] : ib >= 0 ? lb.extent[ib] : lc.extent[ic];
        if (id >= 0 && ld.extent[id] != e)
            return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (label %u)", (long long)e,
                        (long long)ld.extent[id], l);
        if ((ia >= 0 && la.extent[ia] != e) || (ib >= 0 && lb.extent[ib] != e) || (ic >= 0 && lc.extent[ic] != e)) {
            int64_t got = (ib >= 0 && lb.extent[ib] != e) ? lb.extent[ib] : lc.extent[ic >= 0 ? ic : 0];
            return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (label %u)", (long long)e,
                        (long long)got, l);
        }
        Mode m{e, {ia >= 0 ? la.stride[ia] : 0, ib >= 0 ? lb.stride[ib] : 0, ic >= 0 ? lc.stride[ic] : 0,
                   id >= 0 ? ld.stride[id] : 0}};
        if (ic >= 0) {
            if (ia >= 0 && ib >= 0)
                p.batch.push_back(m);
            else if (ia >= 0)
                p.m.push_back(m);
            else if (ib >= 0)
                p.n.push_back(m);
            else
                return fail(TFB_ERR_INVALID_ARGUMENT, "output label %u appears in no input", l);
        } else {
            p.k.push_back(m);  // summed; a label held by one input only meets stride 0 in the other
        }
        return TFB_OK;
    };
    for (auto l : la.labels) TFB_TRY(classify(l));
    for (auto l : lb.labels) TFB_TRY(classify(l));
    for (auto l : lc.labels) TFB_TRY(classify(l));
    // Let the output's fastest-varying free mode be an M mode: the kernels write C along M.
    {
        auto mag = [](int64_t v) { return v < 0 ? -v : v; };
        int64_t best_m = INT64_MAX, best_n = INT64_MAX;
        for (auto& m : p.m)
            if (m.extent > 1 && mag(m.s[2]) < best_m) best_m = mag(m.s[2]);
        for (auto& m : p.n)
            if (m.extent > 1 && mag(m.s[2]) < best_n) best_n = mag(m.s[2]);
        if (best_n < best_m) {
            std::swap(p.a, p.b);
            std::swap(p.conj_a, p.conj_b);
            std::swap(p.m, p.n);
            for (auto* g : {&p.batch, &p.m, &p.n, &p.k})
                for (auto& m : *g) std::swap(m.s[0], m.s[1]);
        }
    }
    sort_and_fuse(p.batch, 2, 4);
    sort_and_fuse(p.m, 0, 4);
    sort_and_fuse(p.n, 1, 4);
    sort_and_fuse(p.k, 0, 4);
    if (algebra != TFB_ALGEBRA_STANDARD) {
        // Tropical semirings have no tensor-core form: every shape, with or without summed labels,
        // runs on the SIMT kernel instantiated for the algebra.
        if (used) *used = "simt_semiring";
        return contract_simt_semiring(ctx, p, algebra);
    }
    if (p.k.empty()) {
        if (d) return fail(TFB_ERR_INVALID_ARGUMENT, "a fused multiplier needs a product with summed labels");
        // No summation: C[b,m,n] = alpha * A[b,m] * B[b,n] + beta * C is element-wise with
        // broadcast strides (Hadamard and outer products; PrimDescriptor::ElementwiseMul).
        std::vector<Mode> all;
        for (auto* g : {&p.m, &p.n, &p.batch})
            for (auto& m : *g) all.push_back(m);
        sort_and_fuse(all, 2, 3);
        LoopNest nest;
        TFB_TRY(make_nest(all, &nest));
        if (used) *used = "elementwise_mul";
        return launch_elementwise_mul(ctx, dtype, nest, p.a, p.b, p.c, alpha, beta, p.conj_a, p.conj_b);
    }
    return launch_contract(ctx, p, force_kernel, used);
}

}  // namespace tfb

using namespace tfb;

// ------------------------------------------------------------------ plan
static tfb_status check_unique(const std::vector<uint32_t>& v, const char* what) {
    std::set<uint32_t> s(v.begin(), v.end());
    if (s.size() != v.size()) return fail(TFB_ERR_INVALID_ARGUMENT, "%s holds a repeated label", what);
    return TFB_OK;
}

static tfb_status check_labels_vs_shapes(const std::vector<std::vector<uint32_t>>& labels,
                                         const std::vector<std::vector<int64_t>>& shapes) {
    std::map<uint32_t, int64_t> ext;
    for (size_t t = 0; t < labels.size(); ++t) {
        if (labels[t].size() != shapes[t].size())
            return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (tensor %zu)", labels[t].size(),
                        shapes[t].size(), t);
        for (size_t i = 0; i < labels[t].size(); ++i) {
            auto it = ext.find(labels[t][i]);
            if (it == ext.end())
                ext[labels[t][i]] = shapes[t][i];
            else if (it->second != shapes[t][i])
                return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (label %u, tensor %zu)",
                            (long long)it->second, (long long)shapes[t][i], labels[t][i], t);
        }
    }
    return TFB_OK;
}

extern "C" {

int tfb_has_extension(int32_t dtype, int32_t ext) {
    // Fused contraction and element-wise multiplication exist for all four Standard types.
    if (!dtype_valid(dtype)) return 0;
    return ext == TFB_EXT_CONTRACT || ext == TFB_EXT_ELEMENTWISE_MUL;
}

tfb_status tfb_plan_create(tfb_ctx* ctx, const tfb_desc* desc, int32_t dtype, size_t n_shapes, const size_t* ranks,
                           const size_t* const* dims, tfb_plan** out) {
    // ctx may be NULL: the plan then only validates and cannot be executed.
    if (!desc || !out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_plan_create: NULL argument");
    *out = nullptr;
    if (!dtype_valid(dtype)) return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", (int)dtype);
    if (n_shapes > 0 && (!ranks || !dims)) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_plan_create: shapes are NULL");
    std::unique_ptr<tfb_plan> p(new tfb_plan);
    p->ctx = ctx;
    p->dtype = dtype;
    p->op = desc->op;
    p->reduce_op = TFB_REDUCE_SUM;
    for (size_t t = 0; t < n_shapes; ++t) {
        std::vector<int64_t> s;
        for (size_t i = 0; i < ranks[t]; ++i) s.push_back((int64_t)dims[t][i]);
        p->shapes.push_back(s);
    }
    auto vec = [](const uint32_t* q, size_t n) { return q ? std::vector<uint32_t>(q, q + n) : std::vector<uint32_t>(); };
    auto need_shapes = [&](size_t n) -> tfb_status {
        if (n_shapes != n)
            return fail(TFB_ERR_INVALID_ARGUMENT, "descriptor needs %zu shapes (inputs first, then output), got %zu", n,
                        n_shapes);
        return TFB_OK;
    };
    // Relabel paired modes: the second label of each pair becomes the first.
    auto apply_pairs = [&](std::vector<uint32_t>& labels, const std::vector<uint32_t>& host) -> tfb_status {
        for (size_t i = 0; i < desc->n_pairs; ++i) {
            uint32_t x = desc->paired[2 * i], y = desc->paired[2 * i + 1];
            if (std::find(host.begin(), host.end(), x) == host.end() ||
                std::find(host.begin(), host.end(), y) == host.end())
                return fail(TFB_ERR_INVALID_ARGUMENT, "paired modes (%u, %u) are not both modes of the paired tensor", x, y);
            if (x == y) return fail(TFB_ERR_INVALID_ARGUMENT, "a mode cannot be paired with itself (%u)", x);
            for (auto& l : labels)
                if (l == y) l = x;
        }
        return TFB_OK;
    };
    switch (desc->op) {
        case TFB_OP_BATCHED_GEMM: {
            TFB_TRY(need_shapes(3));
            const size_t nb = desc->n_batch_dims;
            std::vector<int64_t> ea, eb, ec;
            for (size_t i = 0; i < nb; ++i) {
                ea.push_back((int64_t)desc->batch_dims[i]);
            }
            eb = ec = ea;
            ea.push_back((int64_t)desc->m); ea.push_back((int64_t)desc->k);
            eb.push_back((int64_t)desc->k); eb.push_back((int64_t)desc->n);
            ec.push_back((int64_t)desc->m); ec.push_back((int64_t)desc->n);
            const std::vector<int64_t>* exp[3] = {&ea, &eb, &ec};
            for (int t = 0; t < 3; ++t) {
                if (p->shapes[t].size() != exp[t]->size())
                    return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (tensor %d of BatchedGemm)",
                                exp[t]->size(), p->shapes[t].size(), t);
                if (p->shapes[t] != *exp[t])
                    return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: tensor %d of BatchedGemm is not [batch..., %s]",
                                t, t == 0 ? "m, k" : t == 1 ? "k, n" : "m, n");
            }
            // Labels: batch 3.., m = 0, n = 1, k = 2.
            for (size_t i = 0; i < nb; ++i) {
                p->la.push_back(3 + (uint32_t)i);
                p->lb.push_back(3 + (uint32_t)i);
                p->lc.push_back(3 + (uint32_t)i);
            }
            p->la.push_back(0); p->la.push_back(2);
            p->lb.push_back(2); p->lb.push_back(1);
            p->lc.push_back(0); p->lc.push_back(1);
            p->binary = true;
            break;
        }
        case TFB_OP_CONTRACT: {
            TFB_TRY(need_shapes(3));
            p->la = vec(desc->modes_a, desc->n_modes_a);
            p->lb = vec(desc->modes_b, desc->n_modes_b);
            p->lc = vec(desc->modes_c, desc->n_modes_c);
            TFB_TRY(check_unique(p->lc, "modes_c"));
            TFB_TRY(check_labels_vs_shapes({p->la, p->lb, p->lc}, p->shapes));
            for (auto l : p->lc)
                if (std::find(p->la.begin(), p->la.end(), l) == p->la.end() &&
                    std::find(p->lb.begin(), p->lb.end(), l) == p->lb.end())
                    return fail(TFB_ERR_INVALID_ARGUMENT, "output mode %u appears in neither input", l);
            p->binary = true;
            break;
        }
        case TFB_OP_ELEMENTWISE_MUL: {
            TFB_TRY(need_shapes(3));
            if (p->shapes[0].size() != p->shapes[2].size() || p->shapes[1].size() != p->shapes[2].size())
                return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (ElementwiseMul)",
                            p->shapes[2].size(),
                            p->shapes[0].size() != p->shapes[2].size() ? p->shapes[0].size() : p->shapes[1].size());
            if (p->shapes[0] != p->shapes[2] || p->shapes[1] != p->shapes[2])
                return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: ElementwiseMul needs three equal shapes");
            for (size_t i = 0; i < p->shapes[2].size(); ++i) {
                p->la.push_back((uint32_t)i);
                p->lb.push_back((uint32_t)i);
                p->lc.push_back((uint32_t)i);
            }
            p->binary = true;
            break;
        }
        case TFB_OP_PERMUTE: {
            TFB_TRY(need_shapes(2));
            p->la = vec(desc->modes_a, desc->n_modes_a);
            p->lc = vec(desc->modes_b, desc->n_modes_b);
            TFB_TRY(check_unique(p->la, "modes_a"));
            TFB_TRY(check_unique(p->lc, "modes_b"));
            if (p->la.size() != p->lc.size())
                return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (Permute modes)", p->la.size(),
                            p->lc.size());
            for (auto l : p->lc)
                if (std::find(p->la.begin(), p->la.end(), l) == p->la.end())
                    return fail(TFB_ERR_INVALID_ARGUMENT, "modes_b is not a reordering of modes_a (label %u)", l);
            TFB_TRY(check_labels_vs_shapes({p->la, p->lc}, p->shapes));
            break;
        }
        case TFB_OP_REDUCE: {
            TFB_TRY(need_shapes(2));
            p->la = vec(desc->modes_a, desc->n_modes_a);
            p->lc = vec(desc->modes_c, desc->n_modes_c);
            p->reduce_op = desc->reduce_op;
            if (p->reduce_op < TFB_REDUCE_SUM || p->reduce_op > TFB_REDUCE_MIN)
                return fail(TFB_ERR_INVALID_ARGUMENT, "unknown reduce op %d", p->reduce_op);
            if (p->reduce_op != TFB_REDUCE_SUM && dtype_is_complex(dtype))
                return fail(TFB_ERR_INVALID_ARGUMENT, "Max/Min are undefined for complex types");
            TFB_TRY(check_unique(p->la, "modes_a"));
            TFB_TRY(check_unique(p->lc, "modes_c"));
            for (auto l : p->lc)
                if (std::find(p->la.begin(), p->la.end(), l) == p->la.end())
                    return fail(TFB_ERR_INVALID_ARGUMENT, "modes_c is not a subset of modes_a (label %u)", l);
            TFB_TRY(check_labels_vs_shapes({p->la, p->lc}, p->shapes));
            break;
        }
        case TFB_OP_TRACE: {
            TFB_TRY(need_shapes(2));
            p->la = vec(desc->modes_a, desc->n_modes_a);
            p->lc = vec(desc->modes_c, desc->n_modes_c);
            TFB_TRY(check_unique(p->la, "modes_a"));
            TFB_TRY(check_unique(p->lc, "modes_c"));
            if (desc->n_pairs && !desc->paired) return fail(TFB_ERR_INVALID_ARGUMENT, "paired is NULL");
            std::vector<uint32_t> host = p->la;
            for (size_t i = 0; i < desc->n_pairs; ++i)
                for (int e = 0; e < 2; ++e)
                    if (std::find(p->lc.begin(), p->lc.end(), desc->paired[2 * i + e]) != p->lc.end())
                        return fail(TFB_ERR_INVALID_ARGUMENT, "traced mode %u cannot appear in modes_c",
                                    desc->paired[2 * i + e]);
            for (auto l : p->lc)
                if (std::find(host.begin(), host.end(), l) == host.end())
                    return fail(TFB_ERR_INVALID_ARGUMENT, "modes_c is not a subset of modes_a (label %u)", l);
            TFB_TRY(apply_pairs(p->la, host));
            {
                std::vector<std::vector<uint32_t>> ls = {p->la, p->lc};
                TFB_TRY(check_labels_vs_shapes(ls, p->shapes));
            }
            break;
        }
        case TFB_OP_ANTI_TRACE:
        case TFB_OP_ANTI_DIAG: {
            TFB_TRY(need_shapes(2));
            p->la = vec(desc->modes_a, desc->n_modes_a);
            p->lc = vec(desc->modes_c, desc->n_modes_c);
            TFB_TRY(check_unique(p->la, "modes_a"));
            TFB_TRY(check_unique(p->lc, "modes_c"));
            if (desc->n_pairs && !desc->paired) return fail(TFB_ERR_INVALID_ARGUMENT, "paired is NULL");
            std::vector<uint32_t> host = p->lc;
            // The input may name either label of a pair; both collapse onto the first.
            TFB_TRY(apply_pairs(p->lc, host));
            for (size_t i = 0; i < desc->n_pairs; ++i)
                for (auto& l : p->la)
                    if (l == desc->paired[2 * i + 1]) l = desc->paired[2 * i];
            TFB_TRY(check_unique(p->la, "modes_a (after pairing)"));
            for (auto l : p->la)
                if (std::find(p->lc.begin(), p->lc.end(), l) == p->lc.end())
                    return fail(TFB_ERR_INVALID_ARGUMENT, "input mode %u does not appear in modes_c", l);
            {
                std::vector<std::vector<uint32_t>> ls = {p->la, p->lc};
                TFB_TRY(check_labels_vs_shapes(ls, p->shapes));
            }
            break;
        }
        default:
            return fail(TFB_ERR_INVALID_ARGUMENT, "unknown descriptor op %d", (int)desc->op);
    }
    *out = p.release();
    return TFB_OK;
}

tfb_status tfb_plan_destroy(tfb_plan* plan) {
    delete plan;
    return TFB_OK;
}

const char* tfb_plan_kernel_name(const tfb_plan* plan) { return plan ? plan->kernel_name : "none"; }

static tfb_status check_view_shape(const tfb_view& v, const std::vector<int64_t>& shape, const char* what) {
    if (v.rank != shape.size())
        return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (%s)", shape.size(), v.rank, what);
    for (size_t i = 0; i < shape.size(); ++i)
        if ((int64_t)v.dims[i] != shape[i])
            return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] on axis %zu (%s)",
                        (long long)shape[i], (long long)v.dims[i], i, what);
    return TFB_OK;
}

tfb_status tfb_execute(tfb_plan* plan, const void* alpha, size_t n_inputs, const tfb_view* inputs, const void* beta,
                       const tfb_view* output) {
    if (!plan || !inputs || !output) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_execute: NULL argument");
    if (!alpha || !beta) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_execute: alpha/beta are NULL");
    if (!plan->ctx) return fail(TFB_ERR_INVALID_ARGUMENT, "this plan was created without a context and cannot run");
    const size_t want = plan->binary ? 2 : 1;
    if (n_inputs != want)
        return fail(TFB_ERR_INVALID_ARGUMENT, "this plan takes %zu input(s), got %zu", want, n_inputs);
    Scalar a = load_scalar(plan->dtype, alpha), b = load_scalar(plan->dtype, beta);
    DeviceGuard g(plan->ctx->device);
    const char* used = "none";
    tfb_status st;
    if (plan->binary) {
        TFB_TRY(check_view_shape(inputs[0], plan->shapes[0], "first input"));
        TFB_TRY(check_view_shape(inputs[1], plan->shapes[1], "second input"));
        TFB_TRY(check_view_shape(*output, plan->shapes[2], "output"));
        HView va, vb, vc;
        TFB_TRY(to_hview(inputs[0], plan->dtype, &va, "first input"));
        TFB_TRY(to_hview(inputs[1], plan->dtype, &vb, "second input"));
        TFB_TRY(to_hview(*output, plan->dtype, &vc, "output"));
        st = run_binary(plan->ctx, plan->dtype, plan->la, va, plan->lb, vb, plan->lc, vc, a, b, plan->force_kernel,
                        &used, nullptr, nullptr, plan->algebra);
    } else if (plan->algebra != TFB_ALGEBRA_STANDARD) {
        // One input over a tropical semiring: the same contraction with the semiring's ONE as the
        // second operand - a single element without labels.  One is 0.0 in MaxPlus and MinPlus,
        // i.e. all bits zero.  Reduce(Sum) becomes a maximum (minimum) over the reduced modes,
        // Permute and Trace their semiring forms; alpha and beta combine by (x) = + and (+) = max.
        if (plan->op == TFB_OP_REDUCE && plan->reduce_op != TFB_REDUCE_SUM)
            return fail(TFB_ERR_INVALID_ARGUMENT, "over MaxPlus/MinPlus a Reduce sums with the algebra's own addition: use ReduceOp::Sum");
        TFB_TRY(check_view_shape(inputs[0], plan->shapes[0], "input"));
        TFB_TRY(check_view_shape(*output, plan->shapes[1], "output"));
        HView vi, vo, one;
        TFB_TRY(to_hview(inputs[0], plan->dtype, &vi, "input"));
        TFB_TRY(to_hview(*output, plan->dtype, &vo, "output"));
        PoolBlock unit;
        TFB_TRY(unit.alloc(plan->ctx, 16));
        TFB_CUDA(cudaMemsetAsync(unit.ptr, 0, 16, plan->ctx->stream));
        one.ptr = (char*)unit.ptr;
        st = run_binary(plan->ctx, plan->dtype, plan->la, vi, {}, one, plan->lc, vo, a, b, 0, &used, nullptr, nullptr,
                        plan->algebra);
    } else {
        TFB_TRY(check_view_shape(inputs[0], plan->shapes[0], "input"));
        TFB_TRY(check_view_shape(*output, plan->shapes[1], "output"));
        HView vi, vo;
        TFB_TRY(to_hview(inputs[0], plan->dtype, &vi, "input"));
        TFB_TRY(to_hview(*output, plan->dtype, &vo, "output"));
        st = run_unary(plan->ctx, plan->dtype, plan->la, vi, plan->lc, vo, a, b, plan->reduce_op, &used);
    }
    plan->kernel_name = used;
    return st;
}

tfb_status tfb_plan_set_algebra(tfb_plan* plan, int32_t algebra) {
    if (!plan) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_plan_set_algebra: plan is NULL");
    if (algebra < TFB_ALGEBRA_STANDARD || algebra > TFB_ALGEBRA_MIN_PLUS)
        return fail(TFB_ERR_INVALID_ARGUMENT, "unknown algebra %d", (int)algebra);
    if (algebra != TFB_ALGEBRA_STANDARD) {
        if (plan->dtype != TFB_F32 && plan->dtype != TFB_F64)
            return fail(TFB_ERR_INVALID_ARGUMENT, "MaxPlus and MinPlus are defined for f32 and f64");
        if (plan->op == TFB_OP_ANTI_TRACE || plan->op == TFB_OP_ANTI_DIAG)
            return fail(TFB_ERR_INVALID_ARGUMENT, "AntiTrace and AntiDiag are implemented for the Standard algebra only");
    }
    plan->algebra = algebra;
    return TFB_OK;
}

int tfb_has_extension_for_algebra(int32_t algebra, int32_t dtype, int32_t ext) {
    if (algebra == TFB_ALGEBRA_STANDARD) return tfb_has_extension(dtype, ext);
    if (algebra != TFB_ALGEBRA_MAX_PLUS && algebra != TFB_ALGEBRA_MIN_PLUS) return 0;
    if (dtype != TFB_F32 && dtype != TFB_F64) return 0;
    return ext == TFB_EXT_CONTRACT || ext == TFB_EXT_ELEMENTWISE_MUL;
}

tfb_status tfb_plan_force_kernel(tfb_plan* plan, int kernel) {
    if (!plan) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_plan_force_kernel: plan is NULL");
    plan->force_kernel = kernel;
    return TFB_OK;
}

}  // extern "C"
