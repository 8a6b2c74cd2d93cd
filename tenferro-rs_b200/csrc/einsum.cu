// tenferro-einsum on the device: subscripts, contraction tree, and the tree executor that
// keeps every intermediate in the context's pool.
// Reference: tenferro-einsum/src/lib.rs:239-284 (Subscripts::{new, parse}), :297-356
// (ContractionTree::{optimize, from_pairs}), :393-621 (the nine einsum entry points; the
// accumulating `einsum_with_plan_into` is the one all others reduce to).
#include <algorithm>
#include <cctype>
#include <cmath>
#include <functional>
#include <set>

#include <nvtx3/nvToolsExt.h>

#include "prims.h"

// One NVTX range per tree node, so a timeline shows which kernels belong to which pairwise
// contraction.  Without a profiler attached the calls return at once; TFB_NVTX=0 removes them.
struct NodeRange {
    bool on;
    NodeRange(bool enabled, size_t step, size_t lhs, size_t rhs, bool fused) : on(enabled) {
        if (!on) return;
        char name[96];
        snprintf(name, sizeof name, "tfb einsum node %zu: (%zu, %zu)%s", step, lhs, rhs, fused ? " + fused multiply" : "");
        nvtxRangePushA(name);
    }
    ~NodeRange() {
        if (on) nvtxRangePop();
    }
};

// Nesting of operands given by parentheses: a leaf is an input index, a group is a list.
struct Nest {
    int leaf = -1;
    std::vector<Nest> kids;
};

struct tfb_subscripts {
    std::vector<std::vector<uint32_t>> inputs;
    std::vector<uint32_t> output;
    Nest nest;  // top level: a group of all inputs (possibly nested)
    bool has_parens = false;
};

struct TreeStep {
    size_t lhs, rhs;                // operand ids; intermediates count from n_inputs
    std::vector<uint32_t> labels;   // labels of the result, in storage order
};

struct tfb_tree {
    tfb_subscripts subs;
    std::vector<std::vector<int64_t>> shapes;
    std::map<uint32_t, int64_t> extent;
    std::vector<TreeStep> steps;
    double macs = 0;
};

using namespace tfb;

// ------------------------------------------------------------------ parsing
namespace {

struct Parser {
    const char* s;
    size_t pos = 0;
    tfb_subscripts* out;
    std::string err;

    char peek() {
        while (s[pos] == ' ' || s[pos] == '\t') ++pos;
        return s[pos];
    }
    static bool label_of(char c, uint32_t* l) {
        if (c >= 'a' && c <= 'z') { *l = (uint32_t)(c - 'a'); return true; }
        if (c >= 'A' && c <= 'Z') { *l = 26u + (uint32_t)(c - 'A'); return true; }
        return false;
    }
    // list := item (',' item)* ; item := '(' list ')' | letters*
    bool list(Nest* group, bool top) {
        for (;;) {
            char c = peek();
            if (c == '(') {
                ++pos;
                out->has_parens = true;
                Nest g;
                if (!list(&g, false)) return false;
                if (peek() != ')') { err = "missing ')'"; return false; }
                ++pos;
                if (g.kids.size() == 1) group->kids.push_back(g.kids[0]);
                else group->kids.push_back(g);
            } else {
                std::vector<uint32_t> labels;
                uint32_t l;
                while (label_of(peek(), &l)) { labels.push_back(l); ++pos; }
                Nest leaf;
                leaf.leaf = (int)out->inputs.size();
                out->inputs.push_back(labels);
                group->kids.push_back(leaf);
            }
            c = peek();
            if (c == ',') { ++pos; continue; }
            if (c == ')' && !top) return true;
            if (c == 0 || c == '-') return top ? true : (err = "missing ')'", false);
            err = std::string("unexpected character '") + c + "'";
            return false;
        }
    }
};

}  // namespace

extern "C" {

tfb_status tfb_subscripts_new(size_t n_inputs, const size_t* input_ranks, const uint32_t* const* inputs,
                              size_t output_rank, const uint32_t* output, tfb_subscripts** out) {
    if (!out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_subscripts_new: out is NULL");
    std::unique_ptr<tfb_subscripts> s(new tfb_subscripts);
    for (size_t i = 0; i < n_inputs; ++i) {
        s->inputs.emplace_back(inputs[i], inputs[i] + input_ranks[i]);
        Nest leaf;
        leaf.leaf = (int)i;
        s->nest.kids.push_back(leaf);
    }
    if (output_rank) s->output.assign(output, output + output_rank);
    *out = s.release();
    return TFB_OK;
}

tfb_status tfb_subscripts_parse(const char* notation, tfb_subscripts** out) {
    if (!notation || !out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_subscripts_parse: NULL argument");
    std::unique_ptr<tfb_subscripts> s(new tfb_subscripts);
    Parser p{notation, 0, s.get(), ""};
    if (!p.list(&s->nest, true)) return fail(TFB_ERR_INVALID_ARGUMENT, "malformed einsum notation \"%s\": %s", notation, p.err.c_str());
    if (p.peek() == '-') {
        ++p.pos;
        if (notation[p.pos] != '>') return fail(TFB_ERR_INVALID_ARGUMENT, "malformed einsum notation \"%s\": expected '->'", notation);
        ++p.pos;
        uint32_t l;
        while (Parser::label_of(p.peek(), &l)) { s->output.push_back(l); ++p.pos; }
        if (p.peek() != 0)
            return fail(TFB_ERR_INVALID_ARGUMENT, "malformed einsum notation \"%s\": unexpected character '%c' in the output",
                        notation, p.peek());
    } else {
        // No "->": NumPy's implicit rule - labels seen exactly once, in alphabetical order.
        std::map<uint32_t, int> count;
        for (auto& in : s->inputs)
            for (auto l : in) ++count[l];
        for (auto& kv : count)
            if (kv.second == 1) s->output.push_back(kv.first);
    }
    for (auto l : s->output) {
        bool found = false;
        for (auto& in : s->inputs)
            if (std::find(in.begin(), in.end(), l) != in.end()) found = true;
        if (!found)
            return fail(TFB_ERR_INVALID_ARGUMENT, "malformed einsum notation \"%s\": output label appears in no input", notation);
    }
    *out = s.release();
    return TFB_OK;
}

tfb_status tfb_subscripts_destroy(tfb_subscripts* subs) {
    delete subs;
    return TFB_OK;
}
size_t tfb_subscripts_n_inputs(const tfb_subscripts* subs) { return subs ? subs->inputs.size() : 0; }
size_t tfb_subscripts_input(const tfb_subscripts* subs, size_t i, uint32_t* labels, size_t cap) {
    if (!subs || i >= subs->inputs.size()) return 0;
    const auto& v = subs->inputs[i];
    for (size_t j = 0; j < v.size() && j < cap && labels; ++j) labels[j] = v[j];
    return v.size();
}
size_t tfb_subscripts_output(const tfb_subscripts* subs, uint32_t* labels, size_t cap) {
    if (!subs) return 0;
    for (size_t j = 0; j < subs->output.size() && j < cap && labels; ++j) labels[j] = subs->output[j];
    return subs->output.size();
}
int tfb_subscripts_has_order(const tfb_subscripts* subs) { return subs && subs->has_parens ? 1 : 0; }

}  // extern "C"

// ------------------------------------------------------------------ tree building
namespace {

using LabelSet = std::vector<uint32_t>;  // unique labels, in order

LabelSet unique_of(const std::vector<uint32_t>& v) {
    LabelSet u;
    for (auto l : v)
        if (std::find(u.begin(), u.end(), l) == u.end()) u.push_back(l);
    return u;
}
bool has(const LabelSet& s, uint32_t l) { return std::find(s.begin(), s.end(), l) != s.end(); }

struct Builder {
    tfb_tree* tree;
    // Live operands: id -> labels.
    std::map<size_t, LabelSet> live;
    size_t next_id;

    double ext(uint32_t l) const { return (double)tree->extent.at(l); }

    // Labels the result of contracting x and y must keep: those needed by the final output or
    // by any other live operand.
    LabelSet result_labels(size_t x, size_t y) const {
        LabelSet keep;
        auto needed = [&](uint32_t l) {
            if (has(tree->subs.output, l)) return true;
            for (auto& kv : live)
                if (kv.first != x && kv.first != y && has(kv.second, l)) return true;
            return false;
        };
        for (auto l : live.at(x))
            if (needed(l)) keep.push_back(l);
        for (auto l : live.at(y))
            if (!has(keep, l) && needed(l)) keep.push_back(l);
        return keep;
    }
    double pair_cost(size_t x, size_t y) const {
        double c = 1;
        LabelSet all = live.at(x);
        for (auto l : live.at(y))
            if (!has(all, l)) all.push_back(l);
        for (auto l : all) c *= ext(l);
        return c;
    }
    size_t contract(size_t x, size_t y) {
        TreeStep st;
        st.lhs = x;
        st.rhs = y;
        st.labels = result_labels(x, y);
        tree->macs += pair_cost(x, y);
        live.erase(x);
        live.erase(y);
        size_t id = next_id++;
        live[id] = st.labels;
        tree->steps.push_back(st);
        return id;
    }

    // Best order for the operands `ids` (all live).  Exact subset search up to 12 operands,
    // greedy beyond.  Returns the id of the single operand left.
    size_t optimise_group(std::vector<size_t> ids) {
        const size_t n = ids.size();
        if (n == 1) return ids[0];
        if (n == 2) return contract(ids[0], ids[1]);
        if (n <= 12) {
            // Labels needed outside the group.
            auto outside_needs = [&](uint32_t l) {
                if (has(tree->subs.output, l)) return true;
                for (auto& kv : live)
                    if (std::find(ids.begin(), ids.end(), kv.first) == ids.end() && has(kv.second, l)) return true;
                return false;
            };
            const uint32_t full = (1u << n) - 1;
            // labels(S): labels of members of S needed by a non-member of S or outside the group.
            std::vector<LabelSet> lab(full + 1);
            for (uint32_t S = 1; S <= full; ++S) {
                LabelSet in_s;
                for (size_t i = 0; i < n; ++i)
                    if (S >> i & 1)
                        for (auto l : live.at(ids[i]))
                            if (!has(in_s, l)) in_s.push_back(l);
                for (auto l : in_s) {
                    bool need = outside_needs(l);
                    for (size_t i = 0; i < n && !need; ++i)
                        if (!(S >> i & 1) && has(live.at(ids[i]), l)) need = true;
                    // A single operand keeps all of its labels.
                    if ((S & (S - 1)) == 0) need = true;
                    if (need) lab[S].push_back(l);
                }
            }
            auto size_of = [&](const LabelSet& s) {
                double c = 1;
                for (auto l : s) c *= ext(l);
                return c;
            };
            std::vector<double> best(full + 1, INFINITY), bsize(full + 1, 0);
            std::vector<uint32_t> split(full + 1, 0);
            for (size_t i = 0; i < n; ++i) best[1u << i] = 0;
            for (uint32_t S = 1; S <= full; ++S) {
                if ((S & (S - 1)) == 0) continue;
                for (uint32_t L = (S - 1) & S; L; L = (L - 1) & S) {
                    uint32_t R = S ^ L;
                    if (L < R) continue;  // unordered pairs once
                    LabelSet all = lab[L];
                    for (auto l : lab[R])
                        if (!has(all, l)) all.push_back(l);
                    double c = best[L] + best[R] + size_of(all);
                    double sz = size_of(lab[L]) + size_of(lab[R]);
                    if (c < best[S] || (c == best[S] && sz < bsize[S])) {
                        best[S] = c;
                        bsize[S] = sz;
                        split[S] = L;
                    }
                }
            }
            // Emit steps bottom-up; keep the operand order of the notation (lower index first).
            std::function<size_t(uint32_t)> emit = [&](uint32_t S) -> size_t {
                if ((S & (S - 1)) == 0) {
                    size_t i = 0;
                    while (!(S >> i & 1)) ++i;
                    return ids[i];
                }
                uint32_t L = split[S], R = S ^ L;
                auto lowest = [](uint32_t m) { return m & (~m + 1); };
                if (lowest(R) < lowest(L)) std::swap(L, R);
                size_t x = emit(L);
                size_t y = emit(R);
                return contract(x, y);
            };
            return emit(full);
        }
        // Greedy: cheapest pair first; ties go to the pair whose result is smallest.
        while (ids.size() > 1) {
            double bc = INFINITY, bs = INFINITY;
            size_t bi = 0, bj = 1;
            for (size_t i = 0; i < ids.size(); ++i)
                for (size_t j = i + 1; j < ids.size(); ++j) {
                    double c = pair_cost(ids[i], ids[j]);
                    double s = 1;
                    for (auto l : result_labels(ids[i], ids[j])) s *= ext(l);
                    if (c < bc || (c == bc && s < bs)) { bc = c; bs = s; bi = i; bj = j; }
                }
            size_t id = contract(ids[bi], ids[bj]);
            ids.erase(ids.begin() + bj);
            ids[bi] = id;
        }
        return ids[0];
    }

    size_t build(const Nest& n) {
        if (n.leaf >= 0) return (size_t)n.leaf;
        std::vector<size_t> ids;
        for (auto& k : n.kids) ids.push_back(build(k));
        return optimise_group(ids);
    }
};

tfb_status init_tree(const tfb_subscripts* subs, const size_t* ranks, const size_t* const* dims, tfb_tree* t) {
    t->subs = *subs;
    const size_t n = subs->inputs.size();
    if (n == 0) return fail(TFB_ERR_INVALID_ARGUMENT, "einsum needs at least one operand");
    if (n > 0 && (!ranks || !dims)) return fail(TFB_ERR_INVALID_ARGUMENT, "shapes are NULL");
    for (size_t i = 0; i < n; ++i) {
        if (ranks[i] != subs->inputs[i].size())
            return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (operand %zu)", subs->inputs[i].size(),
                        ranks[i], i);
        std::vector<int64_t> shape;
        for (size_t d = 0; d < ranks[i]; ++d) {
            uint32_t l = subs->inputs[i][d];
            int64_t e = (int64_t)dims[i][d];
            shape.push_back(e);
            auto it = t->extent.find(l);
            if (it == t->extent.end())
                t->extent[l] = e;
            else if (it->second != e)
                return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (label %u, operand %zu)",
                            (long long)it->second, (long long)e, l, i);
        }
        t->shapes.push_back(shape);
    }
    for (auto l : subs->output)
        if (!t->extent.count(l)) return fail(TFB_ERR_INVALID_ARGUMENT, "output label %u appears in no input", l);
    return TFB_OK;
}

}  // namespace

extern "C" {

tfb_status tfb_tree_optimize(const tfb_subscripts* subs, const size_t* ranks, const size_t* const* dims, tfb_tree** out) {
    if (!subs || !out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_tree_optimize: NULL argument");
    std::unique_ptr<tfb_tree> t(new tfb_tree);
    TFB_TRY(init_tree(subs, ranks, dims, t.get()));
    Builder b{t.get(), {}, subs->inputs.size()};
    for (size_t i = 0; i < subs->inputs.size(); ++i) b.live[i] = unique_of(subs->inputs[i]);
    b.build(t->subs.nest);
    *out = t.release();
    return TFB_OK;
}

tfb_status tfb_tree_from_pairs(const tfb_subscripts* subs, const size_t* ranks, const size_t* const* dims, size_t n_pairs,
                               const size_t* pairs, tfb_tree** out) {
    if (!subs || !out) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_tree_from_pairs: NULL argument");
    if (n_pairs && !pairs) return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_tree_from_pairs: pairs is NULL");
    std::unique_ptr<tfb_tree> t(new tfb_tree);
    TFB_TRY(init_tree(subs, ranks, dims, t.get()));
    const size_t n = subs->inputs.size();
    if (n_pairs + 1 != n)
        return fail(TFB_ERR_INVALID_ARGUMENT, "%zu operands need %zu pairwise contractions, got %zu", n, n - 1, n_pairs);
    Builder b{t.get(), {}, n};
    for (size_t i = 0; i < n; ++i) b.live[i] = unique_of(subs->inputs[i]);
    for (size_t s = 0; s < n_pairs; ++s) {
        size_t x = pairs[2 * s], y = pairs[2 * s + 1];
        if (x == y || !b.live.count(x) || !b.live.count(y))
            return fail(TFB_ERR_INVALID_ARGUMENT,
                        "pair %zu = (%zu, %zu) does not name two distinct operands that are still to be contracted", s, x, y);
        b.contract(x, y);
    }
    *out = t.release();
    return TFB_OK;
}

tfb_status tfb_tree_destroy(tfb_tree* tree) {
    delete tree;
    return TFB_OK;
}
size_t tfb_tree_n_steps(const tfb_tree* tree) { return tree ? tree->steps.size() : 0; }
size_t tfb_tree_pairs(const tfb_tree* tree, size_t* pairs, size_t cap) {
    if (!tree) return 0;
    for (size_t s = 0; s < tree->steps.size() && s < cap && pairs; ++s) {
        pairs[2 * s] = tree->steps[s].lhs;
        pairs[2 * s + 1] = tree->steps[s].rhs;
    }
    return tree->steps.size();
}
double tfb_tree_macs(const tfb_tree* tree) { return tree ? tree->macs : 0; }
size_t tfb_tree_output_dims(const tfb_tree* tree, size_t* dims, size_t cap) {
    if (!tree) return 0;
    const auto& o = tree->subs.output;
    for (size_t i = 0; i < o.size() && i < cap && dims; ++i) dims[i] = (size_t)tree->extent.at(o[i]);
    return o.size();
}

// ------------------------------------------------------------------ executor
tfb_status tfb_einsum_with_plan_into(tfb_ctx* ctx, const tfb_tree* tree, int32_t dtype, size_t n_operands,
                                     const tfb_view* operands, const void* alpha, const void* beta, const tfb_view* output) {
    if (!ctx || !tree || !operands || !output || !alpha || !beta)
        return fail(TFB_ERR_INVALID_ARGUMENT, "tfb_einsum_with_plan_into: NULL argument");
    if (!dtype_valid(dtype)) return fail(TFB_ERR_INVALID_ARGUMENT, "unknown dtype %d", (int)dtype);
    const size_t n = tree->subs.inputs.size();
    if (n_operands != n) return fail(TFB_ERR_INVALID_ARGUMENT, "the tree was built for %zu operands, got %zu", n, n_operands);
    DeviceGuard guard(ctx->device);
    const size_t es = dtype_size(dtype);
    const Scalar a = load_scalar(dtype, alpha), b = load_scalar(dtype, beta);
    const Scalar one{1.0, 0.0}, zero{0.0, 0.0};

    // Operand shapes must be the ones the tree was built for.
    for (size_t i = 0; i < n; ++i) {
        if (operands[i].rank != tree->shapes[i].size())
            return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (operand %zu)", tree->shapes[i].size(),
                        operands[i].rank, i);
        for (size_t d = 0; d < operands[i].rank; ++d)
            if ((int64_t)operands[i].dims[d] != tree->shapes[i][d])
                return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (operand %zu, axis %zu)",
                            (long long)tree->shapes[i][d], (long long)operands[i].dims[d], i, d);
    }
    const auto& out_labels = tree->subs.output;
    if (output->rank != out_labels.size())
        return fail(TFB_ERR_RANK_MISMATCH, "rank mismatch: expected %zu, got %zu (output)", out_labels.size(), output->rank);
    for (size_t d = 0; d < out_labels.size(); ++d)
        if ((int64_t)output->dims[d] != tree->extent.at(out_labels[d]))
            return fail(TFB_ERR_SHAPE_MISMATCH, "shape mismatch: expected [%lld], got [%lld] (output axis %zu)",
                        (long long)tree->extent.at(out_labels[d]), (long long)output->dims[d], d);
    HView vout;
    TFB_TRY(to_hview(*output, dtype, &vout, "output"));

    struct Live {
        HView view;
        std::vector<uint32_t> labels;
        std::shared_ptr<PoolBlock> block;  // owning block of an intermediate
    };
    std::map<size_t, Live> live;
    for (size_t i = 0; i < n; ++i) {
        Live l;
        TFB_TRY(to_hview(operands[i], dtype, &l.view, "operand"));
        l.labels = tree->subs.inputs[i];
        live[i] = l;
    }
    const char* used = nullptr;
    if (n == 1) {
        return run_unary(ctx, dtype, live[0].labels, live[0].view, out_labels, vout, a, b, TFB_REDUCE_SUM, &used);
    }
    // Column-major intermediate with the given labels.
    auto make_temp = [&](const std::vector<uint32_t>& labels, Live* l) -> tfb_status {
        l->labels = labels;
        l->view.dims.clear();
        l->view.strides.clear();
        int64_t count = 1;
        for (auto lab : labels) {
            int64_t e = tree->extent.at(lab);
            l->view.dims.push_back(e);
            l->view.strides.push_back(count);
            count *= e;
        }
        l->block = std::make_shared<PoolBlock>();
        TFB_TRY(l->block->alloc(ctx, (size_t)count * es));
        l->view.ptr = (char*)l->block->ptr;
        l->view.conj = false;
        return TFB_OK;
    };
    // Labels an operand holds that nothing else needs are summed away first: it shrinks the
    // operand instead of widening the contraction.
    auto presum = [&](size_t id, size_t partner) -> tfb_status {
        Live& l = live[id];
        std::vector<uint32_t> keep;
        bool drop = false;
        for (auto lab : unique_of(l.labels)) {
            bool needed = has(out_labels, lab);
            for (auto& kv : live)
                if (kv.first != id && has(unique_of(kv.second.labels), lab)) needed = true;
            (void)partner;
            if (needed) keep.push_back(lab);
            else drop = true;
        }
        if (!drop) return TFB_OK;
        Live t;
        TFB_TRY(make_temp(keep, &t));
        TFB_TRY(run_unary(ctx, dtype, l.labels, l.view, t.labels, t.view, one, zero, TFB_REDUCE_SUM, &used));
        live[id] = t;
        return TFB_OK;
    };

    // Label order of the intermediate of step s.  Default: the tree's order.  For Complex32 the
    // labels its consumer will contract go first, in the memory order of the consumer's other
    // operand: the consumer then finds the intermediate with unit stride along K and can feed it
    // to the tensor cores in place instead of copying it (contract_c32.cu).  Only when the
    // leading label is long enough for the producer's writes to stay coalesced.
    auto temp_order = [&](size_t s) -> std::vector<uint32_t> {
        const std::vector<uint32_t>& labs = tree->steps[s].labels;
        if (dtype != TFB_C32) return labs;
        const size_t id = n + s;
        for (size_t c = s + 1; c < tree->steps.size(); ++c) {
            const TreeStep& cs = tree->steps[c];
            if (cs.lhs != id && cs.rhs != id) continue;
            const size_t partner = cs.lhs == id ? cs.rhs : cs.lhs;
            const std::vector<uint32_t>& kept = (c + 1 == tree->steps.size()) ? out_labels : cs.labels;
            std::vector<std::pair<int64_t, uint32_t>> by_stride;
            if (live.count(partner)) {
                const Live& pl = live[partner];
                for (size_t d = 0; d < pl.labels.size(); ++d) by_stride.push_back({std::llabs(pl.view.strides[d]), pl.labels[d]});
            } else if (partner >= n) {
                const auto& pls = tree->steps[partner - n].labels;
                for (size_t d = 0; d < pls.size(); ++d) by_stride.push_back({(int64_t)d, pls[d]});
            }
            std::stable_sort(by_stride.begin(), by_stride.end(),
                             [](const auto& x, const auto& y) { return x.first < y.first; });
            std::vector<uint32_t> order;
            for (const auto& sl : by_stride)
                if (has(labs, sl.second) && !has(kept, sl.second) && !has(order, sl.second)) order.push_back(sl.second);
            if (order.empty() || tree->extent.at(order[0]) < 32) return labs;
            for (auto lab : labs)
                if (!has(order, lab)) order.push_back(lab);
            return order;
        }
        return labs;
    };

    // A product whose only consumer multiplies it element-wise by a tensor that is already at
    // hand (a tree node without summed labels, over the product's own labels) runs as ONE
    // kernel: the multiplier is applied in the product's epilogue and the result goes straight
    // to the consumer's destination.  Returns the consumer's step, or 0.
    const bool fuse_mul = env_int("TFB_EINSUM_FUSE_MUL", 1) != 0;
    auto fusable_consumer = [&](size_t s, const Live& x, const Live& y) -> size_t {
        if (!fuse_mul) return 0;
        const TreeStep& st = tree->steps[s];
        const size_t id = n + s;
        const LabelSet mine = unique_of(st.labels);
        if (mine.size() != st.labels.size()) return 0;
        // The product must really sum something: labels of extent 1 vanish when the modes are
        // fused, and a product without a K group cannot carry a multiplier.
        int64_t summed = 1;
        for (auto lab : unique_of(x.labels))
            if (has(unique_of(y.labels), lab) && !has(mine, lab)) summed *= tree->extent.at(lab);
        if (summed <= 1) return 0;
        for (size_t c = s + 1; c < tree->steps.size(); ++c) {
            const TreeStep& cs = tree->steps[c];
            if (cs.lhs != id && cs.rhs != id) continue;
            const size_t partner = cs.lhs == id ? cs.rhs : cs.lhs;
            if (partner == id || partner == st.lhs || partner == st.rhs || !live.count(partner)) return 0;
            const std::vector<uint32_t>& kept = (c + 1 == tree->steps.size()) ? out_labels : cs.labels;
            const LabelSet kept_set = unique_of(kept);
            if (kept_set.size() != kept.size() || kept_set.size() != mine.size()) return 0;
            for (auto lab : mine)
                if (!has(kept_set, lab)) return 0;
            for (auto lab : live[partner].labels)
                if (!has(mine, lab)) return 0;
            return c;
        }
        return 0;
    };

    std::vector<char> done(tree->steps.size(), 0);
    const bool nvtx = env_int("TFB_NVTX", 1) != 0;
    for (size_t s = 0; s < tree->steps.size(); ++s) {
        if (done[s]) continue;
        const TreeStep& st = tree->steps[s];
        if (!live.count(st.lhs) || !live.count(st.rhs)) return fail(TFB_ERR_INVALID_ARGUMENT, "corrupt contraction tree");
        TFB_TRY(presum(st.lhs, st.rhs));
        TFB_TRY(presum(st.rhs, st.lhs));
        const bool last = s + 1 == tree->steps.size();
        Live& x = live[st.lhs];
        Live& y = live[st.rhs];
        const size_t c = last ? 0 : fusable_consumer(s, x, y);
        NodeRange range(nvtx, s, st.lhs, st.rhs, c != 0);
        if (last) {
            TFB_TRY(run_binary(ctx, dtype, x.labels, x.view, y.labels, y.view, out_labels, vout, a, b, 0, &used));
        } else if (c != 0) {
            const TreeStep& cs = tree->steps[c];
            const size_t partner = cs.lhs == n + s ? cs.rhs : cs.lhs;
            const Live& dmul = live[partner];
            if (c + 1 == tree->steps.size()) {
                TFB_TRY(run_binary(ctx, dtype, x.labels, x.view, y.labels, y.view, out_labels, vout, a, b, 0, &used,
                                   &dmul.labels, &dmul.view));
            } else {
                Live t;
                TFB_TRY(make_temp(temp_order(c), &t));
                TFB_TRY(run_binary(ctx, dtype, x.labels, x.view, y.labels, y.view, t.labels, t.view, one, zero, 0, &used,
                                   &dmul.labels, &dmul.view));
                live[n + c] = t;
            }
            done[c] = 1;
            live.erase(partner);
        } else {
            Live t;
            TFB_TRY(make_temp(temp_order(s), &t));
            TFB_TRY(run_binary(ctx, dtype, x.labels, x.view, y.labels, y.view, t.labels, t.view, one, zero, 0, &used));
            live[n + s] = t;
        }
        // Intermediates go back to the pool in stream order as soon as their consumer is enqueued.
        live.erase(st.lhs);
        live.erase(st.rhs);
    }
    return TFB_OK;
}

}  // extern "C"
