"""The oracle checked against itself and against the known answers: NumPy restatement vs the
C nested-loop restatement vs the fixtures in tests/golden/."""
import json
from pathlib import Path

import numpy as np
import pytest

from conftest import ALL_DTYPES, TOL, Strided, random_array

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN / "golden.npz")


@pytest.fixture(scope="module")
def kat():
    return json.loads((GOLDEN / "kat.json").read_text())


def c_run(oracle, labels_in, arrays, labels_out, out_shape, dtype, alpha=1.0, beta=0.0, out_old=None, op=0, conj=None):
    ins = [oracle.StridedBuf.col_major(a) for a in arrays]
    if conj:
        for sb, cj in zip(ins, conj):
            sb.conj = cj
    init = np.zeros(out_shape, dtype=dtype) if out_old is None else np.asarray(out_old, dtype=dtype)
    out = oracle.StridedBuf.col_major(init)
    oracle.c_execute(labels_in, ins, labels_out, out, alpha, beta, op)
    return np.array(out.view())


def test_kat_from_slice(kat, oracle):
    c = kat["from_slice_2x3"]
    sb = oracle.StridedBuf(np.array(c["data"], dtype=np.float64), c["dims"], [1, 2])
    assert sb.view().tolist() == c["logical"]


@pytest.mark.parametrize("notation", ["ij,jk->ik", "ii->", "i,j->ij", "i,i->", "ij,j->i", "i->ii", "ii->i", "i->iii",
                                      "ij->ji", "ijk->"])
def test_kat_einsum_numpy_and_c(kat, oracle, notation):
    case = kat[notation]
    ops = [np.array(x, dtype=np.float64) for x in case["operands"]]
    want = np.array(case["result"], dtype=np.float64)
    got = oracle.np_einsum(notation, ops)
    assert np.array_equal(got, want)
    ins, out = oracle.parse_notation(notation)
    got_c = c_run(oracle, ins, ops, out, want.shape, np.float64)
    assert np.array_equal(got_c, want)


def test_kat_conj(kat, oracle):
    c = kat["conj"]
    z = np.array([complex(*p) for p in c["operand"]])
    want = np.array([complex(*p) for p in c["result"]])
    assert np.array_equal(np.conj(z), want)
    got = c_run(oracle, [[0]], [z], [0], z.shape, np.complex128, conj=[True])
    assert np.array_equal(got, want)


def test_kat_accumulate(kat, oracle):
    c = kat["accumulate"]
    ops = [np.array(x, dtype=np.float64) for x in c["operands"]]
    out = np.zeros((2, 2))
    for _ in range(2):
        out = oracle.np_einsum(c["notation"], ops, c["alpha"], c["beta"], out)
    assert out.tolist() == c["result_after_two_calls"]


@pytest.mark.parametrize("name,dtype", [("f32", np.float32), ("f64", np.float64), ("c32", np.complex64),
                                        ("c64", np.complex128)])
def test_c_oracle_matches_golden(golden, oracle, name, dtype):
    tol = TOL[np.dtype(dtype)]
    g = golden
    got = c_run(oracle, [[0, 1, 2], [2, 1, 3]], [g[f"contract_{name}_a"], g[f"contract_{name}_b"]], [3, 0], (6, 5), dtype,
                0.5, -2.0, g[f"contract_{name}_c0"])
    assert oracle.rel_frobenius(got, g[f"contract_{name}_out"]) <= tol
    got = c_run(oracle, [[9, 0, 2], [9, 2, 1]], [g[f"bgemm_{name}_a"], g[f"bgemm_{name}_b"]], [9, 0, 1], (4, 3, 2), dtype)
    assert oracle.rel_frobenius(got, g[f"bgemm_{name}_out"]) <= tol
    got = c_run(oracle, [[0, 1, 2]], [g[f"reduce_{name}_a"]], [2, 0], (5, 4), dtype)
    assert oracle.rel_frobenius(got, g[f"reduce_{name}_sum"]) <= tol
    if np.dtype(dtype).kind != "c":
        for key, op in (("max", 1), ("min", 2)):
            got = c_run(oracle, [[0, 1, 2]], [g[f"reduce_{name}_a"]], [1], (6,), dtype, op=op)
            assert np.array_equal(got, g[f"reduce_{name}_{key}"])
    got = c_run(oracle, [[0, 1, 0]], [g[f"trace_{name}_a"]], [1], (3,), dtype)
    assert oracle.rel_frobenius(got, g[f"trace_{name}_out"]) <= tol
    got = c_run(oracle, [[0, 1, 2]], [g[f"permute_{name}_a"]], [2, 0, 1], (5, 3, 4), dtype)
    assert np.array_equal(got, g[f"permute_{name}_out"])
    got = c_run(oracle, [[1]], [g[f"antitrace_{name}_a"]], [0, 1, 0], (4, 3, 4), dtype)
    assert np.array_equal(got, g[f"antitrace_{name}_out"])
    got = c_run(oracle, [[0, 1]], [g[f"antidiag_{name}_a"]], [0, 1, 0], (4, 3, 4), dtype)
    assert np.array_equal(got, g[f"antidiag_{name}_out"])
    got = c_run(oracle, [[0, 1], [0, 1]], [g[f"ewmul_{name}_a"], g[f"ewmul_{name}_b"]], [0, 1], (3, 4), dtype)
    assert oracle.rel_frobenius(got, g[f"ewmul_{name}_out"]) <= tol


def test_c_oracle_benchmark_einsums(golden, oracle):
    g = golden
    got = c_run(oracle, [[0, 1, 2], [1, 2, 3]], [g["cfg1_a"], g["cfg1_b"]], [0, 3], (8, 8), np.float64)
    assert oracle.rel_frobenius(got, g["cfg1_out"]) <= 1e-12
    got = c_run(oracle, [[0, 1, 2, 3], [2, 3, 4, 5]], [g["cfg5_a"], g["cfg5_b"]], [0, 1, 4, 5], (4, 4, 4, 4), np.float32)
    assert oracle.rel_frobenius(got, g["cfg5_out"]) <= 1e-5
    # ttgt (the timed CPU baseline) agrees with the einsum truth
    got = oracle.ttgt_contract([0, 1, 2, 3], g["cfg5_a"], [2, 3, 4, 5], g["cfg5_b"], [0, 1, 4, 5])
    assert oracle.rel_frobenius(got, g["cfg5_out"]) <= 1e-5


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_c_oracle_strided_views(oracle, dtype):
    """Random layouts (permuted, padded, offset, reversed axes) and conj flags: the C loops over
    raw strides agree with NumPy on the logical arrays."""
    rng = np.random.default_rng(11)
    for trial in range(10):
        m, n, k, b = (int(x) for x in rng.integers(1, 6, size=4))
        a = Strided(random_array(rng, (b, m, k), dtype), rng, conj=bool(trial % 2))
        bb = Strided(random_array(rng, (k, b, n), dtype), rng, conj=bool(trial % 3 == 0))
        c = Strided(random_array(rng, (n, m, b), dtype), rng)
        alpha, beta = (0.5, -1.0) if trial % 2 else (1.0, 0.0)
        want = oracle.np_contract([0, 1, 2], a.logical, [2, 0, 3], bb.logical, [3, 1, 0], alpha, beta, c.logical)
        out = c.to_oracle(oracle)
        oracle.c_execute([[0, 1, 2], [2, 0, 3]], [a.to_oracle(oracle), bb.to_oracle(oracle)], [3, 1, 0], out, alpha, beta)
        assert oracle.rel_frobenius(out.view(), want) <= TOL[np.dtype(dtype)]
        # Gaps between elements are untouched.
        mask = np.ones(out.buf.shape, dtype=bool)
        it = out.buf.dtype.itemsize
        idx = np.lib.stride_tricks.as_strided(np.arange(out.buf.size)[out.offset:], shape=out.dims,
                                              strides=[s * 8 for s in out.strides])
        mask[idx.reshape(-1)] = False
        assert np.array_equal(out.buf[mask], c.buf[mask])
