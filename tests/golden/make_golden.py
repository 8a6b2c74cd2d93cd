"""Writes tests/golden/golden.npz and tests/golden/kat.json.

The reference asserts no numbers for this path (its arithmetic is `todo!()`), so these
fixtures come from two sources:
  * kat.json   - hand-checkable answers for the 2x2 / length-3 operands the reference's doc
                 examples use (tenferro-einsum/src/lib.rs:31-63; tenferro-tensor/src/lib.rs:34-39,
                 617-620), worked out with integer arithmetic below;
  * golden.npz - seeded random inputs with float64/complex128 NumPy results for every
                 descriptor and for scaled-down versions of the five benchmark einsums.
Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
from oracle import oracle as o  # noqa: E402


def kat():
    # Column-major from_slice([1..6], [2,3]) is [[1,3,5],[2,4,6]] (tenferro-tensor/src/lib.rs:34-39).
    a = [[1, 3], [2, 4]]  # from_slice([1,2,3,4], [2,2])
    b = [[5, 7], [6, 8]]  # from_slice([5,6,7,8], [2,2])
    v = [1, 2, 3]
    mm = [[sum(a[i][j] * b[j][k] for j in range(2)) for k in range(2)] for i in range(2)]
    cases = {
        "from_slice_2x3": {"data": [1, 2, 3, 4, 5, 6], "dims": [2, 3], "logical": [[1, 3, 5], [2, 4, 6]]},
        "ij,jk->ik": {"operands": [a, b], "result": mm},
        "ii->": {"operands": [a], "result": a[0][0] + a[1][1]},
        "i,j->ij": {"operands": [v, v], "result": [[x * y for y in v] for x in v]},
        "i,i->": {"operands": [v, v], "result": sum(x * x for x in v)},
        "ij,j->i": {"operands": [a, [1, 2]], "result": [a[i][0] * 1 + a[i][1] * 2 for i in range(2)]},
        "i->ii": {"operands": [v], "result": [[v[i] if i == j else 0 for j in range(3)] for i in range(3)]},
        "ii->i": {"operands": [a], "result": [a[0][0], a[1][1]]},
        "i->iii": {"operands": [v],
                   "result": [[[v[i] if i == j == k else 0 for k in range(3)] for j in range(3)] for i in range(3)]},
        "ij->ji": {"operands": [a], "result": [[a[j][i] for j in range(2)] for i in range(2)]},
        "ijk->": {"operands": [[[[1, 2], [3, 4]], [[5, 6], [7, 8]]]], "result": 36},
        "conj": {"operand": [[1.0, 2.0], [3.0, -4.0]], "result": [[1.0, -2.0], [3.0, 4.0]]},
        "accumulate": {"notation": "ij,jk->ik", "operands": [a, b], "alpha": 1.0, "beta": 1.0,
                       "result_after_two_calls": [[2 * x for x in row] for row in mm]},
    }
    (HERE / "kat.json").write_text(json.dumps(cases, indent=1))


def golden():
    out = {}
    rng = np.random.default_rng(20260213)

    def rnd(shape, dtype):
        dtype = np.dtype(dtype)
        if dtype.kind == "c":
            return (rng.standard_normal(shape) + 1j * rng.standard_normal(shape)).astype(dtype)
        return rng.standard_normal(shape).astype(dtype)

    for name, dt in (("f32", np.float32), ("f64", np.float64), ("c32", np.complex64), ("c64", np.complex128)):
        a, b = rnd((5, 7, 3), dt), rnd((3, 7, 6), dt)
        c0 = rnd((6, 5), dt)
        out[f"contract_{name}_a"], out[f"contract_{name}_b"], out[f"contract_{name}_c0"] = a, b, c0
        # C[n,m] = 0.5 * sum_{k,l} A[m,k,l] B[l,k,n] - 2 * C
        out[f"contract_{name}_out"] = o.np_contract([0, 1, 2], a, [2, 1, 3], b, [3, 0], 0.5, -2.0, c0)
        g1, g2 = rnd((4, 3, 5), dt), rnd((4, 5, 2), dt)
        out[f"bgemm_{name}_a"], out[f"bgemm_{name}_b"] = g1, g2
        out[f"bgemm_{name}_out"] = o.np_batched_gemm(g1, g2)
        r = rnd((4, 6, 5), dt)
        out[f"reduce_{name}_a"] = r
        out[f"reduce_{name}_sum"] = o.np_reduce([0, 1, 2], r, [2, 0], 0)
        if np.dtype(dt).kind != "c":
            out[f"reduce_{name}_max"] = o.np_reduce([0, 1, 2], r, [1], 1)
            out[f"reduce_{name}_min"] = o.np_reduce([0, 1, 2], r, [1], 2)
        t = rnd((4, 3, 4), dt)
        out[f"trace_{name}_a"] = t
        out[f"trace_{name}_out"] = o.np_trace([0, 1, 2], t, [1], [(0, 2)])
        p = rnd((3, 4, 5), dt)
        out[f"permute_{name}_a"] = p
        out[f"permute_{name}_out"] = o.np_permute([0, 1, 2], p, [2, 0, 1])
        g = rnd((3,), dt)
        out[f"antitrace_{name}_a"] = g
        out[f"antitrace_{name}_out"] = o.np_anti_trace([1], g, [0, 1, 2], (4, 3, 4), [(0, 2)])
        d = rnd((4, 3), dt)
        out[f"antidiag_{name}_a"] = d
        out[f"antidiag_{name}_out"] = o.np_anti_diag([0, 1], d, [0, 1, 2], (4, 3, 4), [(0, 2)])
        e1, e2 = rnd((3, 4), dt), rnd((3, 4), dt)
        out[f"ewmul_{name}_a"], out[f"ewmul_{name}_b"] = e1, e2
        out[f"ewmul_{name}_out"] = o.np_elementwise_mul(e1, e2)

    # Scaled-down versions of the five benchmark einsums (same notation, same distributions).
    a, b = o.normal(1000, (8, 8, 8), np.float64), o.normal(1001, (8, 8, 8), np.float64)
    out["cfg1_a"], out["cfg1_b"], out["cfg1_out"] = a, b, o.np_einsum("abc,bcd->ad", [a, b])
    chi, d = 16, 2
    e = np.eye(chi, dtype=np.complex128)
    site = o.normal(2000, (chi, d, chi), np.complex128, scale=(1.0 / chi) ** 0.5)
    out["cfg2_e"], out["cfg2_a"] = e, site
    out["cfg2_out"] = o.np_einsum("ab,asc,bsd->cd", [e, site, np.conj(site)])
    table = o.grouped_table(3000, 6)
    out["cfg3_table"] = table
    for p, (i, j, k) in enumerate(table):
        x, y = o.uniform(3001 + 2 * p, (i, j), np.float32), o.uniform(3002 + 2 * p, (j, k), np.float32)
        out[f"cfg3_a{p}"], out[f"cfg3_b{p}"] = x, y
        out[f"cfg3_out{p}"] = o.np_batched_gemm(x, y)
    ops = [o.normal(4000 + i, (6, 6, 6), np.complex64) for i in range(4)]
    for i, t in enumerate(ops):
        out[f"cfg4_op{i}"] = t
    out["cfg4_out"] = o.np_einsum("ijk,jlm,kmn,lnp->ip", ops)
    a, b = o.normal(5000, (4, 4, 8, 8), np.float32), o.normal(5001, (8, 8, 4, 4), np.float32)
    out["cfg5_a"], out["cfg5_b"], out["cfg5_out"] = a, b, o.np_einsum("ijkl,klmn->ijmn", [a, b])
    np.savez_compressed(HERE / "golden.npz", **out)


if __name__ == "__main__":
    kat()
    golden()
    print("wrote", HERE / "kat.json", "and", HERE / "golden.npz")
