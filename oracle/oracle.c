/*
 * oracle.c - CPU restatement of the tenferro-prims operation semantics.  TEST INFRASTRUCTURE:
 * only tests, the smoke check and the benchmark's CPU-baseline leg may call it; nothing in
 * the product path links or loads it.
 *
 * PARITY UNPINNED: the reference holds no executable arithmetic for this path (every body is
 * `todo!()`, tenferro-prims/src/lib.rs:422-438, tenferro-einsum/src/lib.rs:393-621), its CPU
 * kernels live in an un-vendored, un-pinned git dependency (strided-rs,
 * tenferro-prims/Cargo.toml:12-13) and its tests assert no numbers.  What is restated here
 * is therefore the documented semantics, as plain nested loops over signed element strides:
 *
 *   execute contract         output = alpha * op(inputs) + beta * output
 *                            (tenferro-prims/src/lib.rs:300-303)
 *   mode rule                modes shared by inputs and output are batch/free, modes only in
 *                            inputs are summed (tenferro-prims/src/lib.rs:136-138)
 *   Contract / BatchedGemm   :156-168, :227-239
 *   Reduce (Sum/Max/Min)     :170-180
 *   Trace / AntiTrace / AntiDiag  :182-222 (a label repeated inside one tensor walks its
 *                            diagonal: both axes advance together)
 *   Permute                  :194-202
 *   ElementwiseMul           :241-244
 *   conj                     tenferro-tensor/src/lib.rs:606-647 (negate the imaginary part)
 *
 * Sums are accumulated in double (complex double) whatever the element type, so for f32 and
 * Complex32 this is the exact-arithmetic answer rounded once.
 *
 * dtype codes: 0 f32, 1 f64, 2 Complex32, 3 Complex64.  Pointers are element pointers (any
 * offset already applied); strides count elements.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MAXL 32

typedef struct {
    double re, im;
} cplx;

static cplx load(int dtype, const void* p, int64_t off, int conj) {
    cplx v = {0, 0};
    switch (dtype) {
        case 0: v.re = ((const float*)p)[off]; break;
        case 1: v.re = ((const double*)p)[off]; break;
        case 2: v.re = ((const float*)p)[2 * off]; v.im = ((const float*)p)[2 * off + 1]; break;
        case 3: v.re = ((const double*)p)[2 * off]; v.im = ((const double*)p)[2 * off + 1]; break;
    }
    if (conj) v.im = -v.im;
    return v;
}

static void store(int dtype, void* p, int64_t off, cplx v) {
    switch (dtype) {
        case 0: ((float*)p)[off] = (float)v.re; break;
        case 1: ((double*)p)[off] = v.re; break;
        case 2: ((float*)p)[2 * off] = (float)v.re; ((float*)p)[2 * off + 1] = (float)v.im; break;
        case 3: ((double*)p)[2 * off] = v.re; ((double*)p)[2 * off + 1] = v.im; break;
    }
}

static cplx cmul(cplx a, cplx b) {
    cplx r = {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re};
    return r;
}

/* Label table: unique labels with extent and the summed stride each tensor gives them. */
typedef struct {
    int n;
    uint32_t label[MAXL];
    int64_t extent[MAXL];
    int64_t stride[3][MAXL];
    int in_tensor[3][MAXL];
} table;

static int add_labels(table* t, int which, int rank, const int64_t* dims, const int64_t* strides,
                      const uint32_t* labels) {
    for (int i = 0; i < rank; ++i) {
        int j;
        for (j = 0; j < t->n; ++j)
            if (t->label[j] == labels[i]) break;
        if (j == t->n) {
            if (t->n == MAXL) return -1;
            t->label[j] = labels[i];
            t->extent[j] = dims[i];
            for (int w = 0; w < 3; ++w) {
                t->stride[w][j] = 0;
                t->in_tensor[w][j] = 0;
            }
            t->n++;
        } else if (t->extent[j] != dims[i]) {
            return -2;
        }
        t->stride[which][j] += strides[i];
        t->in_tensor[which][j] = 1;
    }
    return 0;
}

/* Scale every element of a strided tensor by beta (used when the output has repeated labels:
 * off-diagonal elements only see beta). */
static void scale_all(int dtype, void* p, int rank, const int64_t* dims, const int64_t* strides, cplx beta) {
    int64_t idx[MAXL] = {0};
    int64_t total = 1;
    for (int i = 0; i < rank; ++i) total *= dims[i];
    for (int64_t n = 0; n < total; ++n) {
        int64_t off = 0;
        for (int i = 0; i < rank; ++i) off += idx[i] * strides[i];
        cplx v = {0, 0};
        if (beta.re != 0 || beta.im != 0) v = cmul(beta, load(dtype, p, off, 0));
        store(dtype, p, off, v);
        for (int i = 0; i < rank; ++i) {
            if (++idx[i] < dims[i]) break;
            idx[i] = 0;
        }
    }
}

static int has_repeats(int rank, const uint32_t* labels) {
    for (int i = 0; i < rank; ++i)
        for (int j = i + 1; j < rank; ++j)
            if (labels[i] == labels[j]) return 1;
    return 0;
}

/*
 * C[labels_c] = alpha * sum_{labels not in C} A[labels_a] * B[labels_b] + beta * C.
 * With n_inputs == 1 (b == NULL) the product is just A and `reduce_op` (0 sum, 1 max, 2 min)
 * combines the values over the labels missing from C.
 * Returns 0, or a negative code for inconsistent extents / too many labels / bad output label.
 */
int oracle_execute(int dtype, int n_inputs,
                   int rank_a, const int64_t* dims_a, const int64_t* strides_a, const uint32_t* labels_a,
                   const void* a, int conj_a,
                   int rank_b, const int64_t* dims_b, const int64_t* strides_b, const uint32_t* labels_b,
                   const void* b, int conj_b,
                   int rank_c, const int64_t* dims_c, const int64_t* strides_c, const uint32_t* labels_c, void* c,
                   const double* alpha2, const double* beta2, int reduce_op) {
    table t;
    t.n = 0;
    int rc;
    if ((rc = add_labels(&t, 0, rank_a, dims_a, strides_a, labels_a))) return rc;
    if (n_inputs == 2 && (rc = add_labels(&t, 1, rank_b, dims_b, strides_b, labels_b))) return rc;
    const int n_in_labels = t.n;
    if ((rc = add_labels(&t, 2, rank_c, dims_c, strides_c, labels_c))) return rc;
    /* Broadcast (a label only in the output) is allowed for the unary form only. */
    if (n_inputs == 2 && t.n != n_in_labels) return -3;
    cplx alpha = {alpha2[0], alpha2[1]}, beta = {beta2[0], beta2[1]};
    if (has_repeats(rank_c, labels_c)) {
        scale_all(dtype, c, rank_c, dims_c, strides_c, beta);
        if (beta.re != 0 || beta.im != 0) {
            beta.re = 1;
            beta.im = 0;
        }
    }
    /* Split labels into kept (in C) and summed. */
    int kept[MAXL], nk = 0, red[MAXL], nr = 0;
    for (int j = 0; j < t.n; ++j) {
        if (t.in_tensor[2][j]) kept[nk++] = j;
        else red[nr++] = j;
    }
    int64_t total_k = 1, total_r = 1;
    for (int i = 0; i < nk; ++i) total_k *= t.extent[kept[i]];
    for (int i = 0; i < nr; ++i) total_r *= t.extent[red[i]];
    if (total_r == 0 && reduce_op != 0) return -4;
    int64_t ik[MAXL] = {0};
    for (int64_t nko = 0; nko < total_k; ++nko) {
        int64_t oa = 0, ob = 0, oc = 0;
        for (int i = 0; i < nk; ++i) {
            oa += ik[i] * t.stride[0][kept[i]];
            ob += ik[i] * t.stride[1][kept[i]];
            oc += ik[i] * t.stride[2][kept[i]];
        }
        cplx acc = {0, 0};
        int first = 1;
        int64_t ir[MAXL] = {0};
        for (int64_t nro = 0; nro < total_r; ++nro) {
            int64_t ra = oa, rb = ob;
            for (int i = 0; i < nr; ++i) {
                ra += ir[i] * t.stride[0][red[i]];
                rb += ir[i] * t.stride[1][red[i]];
            }
            cplx v = load(dtype, a, ra, conj_a);
            if (n_inputs == 2) v = cmul(v, load(dtype, b, rb, conj_b));
            if (reduce_op == 0) {
                acc.re += v.re;
                acc.im += v.im;
            } else if (first) {
                acc = v;
            } else if (isnan(acc.re)) {
                /* NaN sticks */
            } else if (isnan(v.re) || (reduce_op == 1 ? v.re > acc.re : v.re < acc.re)) {
                acc = v;
            }
            first = 0;
            for (int i = 0; i < nr; ++i) {
                if (++ir[i] < t.extent[red[i]]) break;
                ir[i] = 0;
            }
        }
        cplx out = cmul(alpha, acc);
        if (beta.re != 0 || beta.im != 0) {
            cplx old = cmul(beta, load(dtype, c, oc, 0));
            out.re += old.re;
            out.im += old.im;
        }
        store(dtype, c, oc, out);
        for (int i = 0; i < nk; ++i) {
            if (++ik[i] < t.extent[kept[i]]) break;
            ik[i] = 0;
        }
    }
    return 0;
}
