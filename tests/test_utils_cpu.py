"""CPU: CSR helpers (conversion, transpose bookkeeping, partitioning, row split)."""
import numpy as np
import torch

from intrasm_engine_b200.pytorch import utils as U


def _rand_dense(m, k, density, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(m, k, generator=g) * (torch.rand(m, k, generator=g) < density)


def test_dense_to_sparse_roundtrip_and_order():
    d = _rand_dense(37, 53, 0.3)
    v, ri, ro, ci = U.dense_to_sparse(d)
    assert ri.dtype == torch.int32 and ro.dtype == torch.int32 and ci.dtype == torch.int32
    assert torch.equal(U.sparse_to_dense(v, ro, ci, 37, 53), d)
    counts = (ro[1:] - ro[:-1])[ri.long()]
    assert torch.all(counts[:-1] >= counts[1:])
    for r in range(37):
        seg = ci[ro[r]:ro[r + 1]]
        assert torch.all(seg[1:] > seg[:-1])
    v16, _, _, ci16 = U.dense_to_sparse(d.half(), index_dtype=torch.int16)
    assert ci16.dtype == torch.int16 and v16.dtype == torch.float16


def test_matches_host_generator(oracle):
    from intrasm_engine_b200 import synthetic as syn
    d = _rand_dense(20, 31, 0.4, 3)
    a = syn.dense_to_csr(d.numpy())
    v, ri, ro, ci = U.dense_to_sparse(d)
    np.testing.assert_array_equal(a.values, v.numpy())
    np.testing.assert_array_equal(a.row_offsets, ro.numpy())
    np.testing.assert_array_equal(a.column_indices, ci.numpy())
    np.testing.assert_array_equal(a.row_indices, ri.numpy())
    assert oracle.validate_csr(20, 31, ri.numpy(), ro.numpy(), ci.numpy()) == 0


def test_transpose_info():
    d = _rand_dense(29, 17, 0.35, 1)
    v, ri, ro, ci = U.dense_to_sparse(d)
    info = U.get_transpose_info(29, 17, ri, ro, ci)
    ri_t, v_t, ro_t, ci_t = U.transpose_with_info(v, info)
    assert torch.equal(U.sparse_to_dense(v_t, ro_t, ci_t, 17, 29), d.t())
    for r in range(17):
        seg = ci_t[ro_t[r]:ro_t[r + 1]]
        assert torch.all(seg[1:] > seg[:-1])
    # new values, same pattern: only the permutation is applied
    v2 = torch.randn_like(v)
    _, v2_t, _, _ = U.transpose_with_info(v2, info)
    assert torch.equal(U.sparse_to_dense(v2_t, ro_t, ci_t, 17, 29), U.sparse_to_dense(v2, ro, ci, 29, 17).t())


def test_partition_csr_and_coo():
    d = _rand_dense(12, 16, 0.5, 2)
    v, ri, ro, ci = U.dense_to_sparse(d)
    crow, col, val = U.partition_csr(ro.long(), ci.long(), v, 12, 16, 4, 8)
    assert len(crow) == 3 and len(crow[0]) == 2
    for i in range(3):
        for j in range(2):
            blk = U.sparse_to_dense(val[i][j], crow[i][j], col[i][j], 4, 8)
            assert torch.equal(blk, d[4 * i:4 * i + 4, 8 * j:8 * j + 8])
    rows = torch.repeat_interleave(torch.arange(12), (ro[1:] - ro[:-1]).long())
    r, c, vv = U.partition_coo(rows, ci, v, 12, 16, 6, 4)
    for i in range(2):
        for j in range(4):
            blk = torch.zeros(6, 4)
            blk[r[i][j], c[i][j]] = vv[i][j]
            assert torch.equal(blk, d[6 * i:6 * i + 6, 4 * j:4 * j + 4])


def test_nnz_balanced_row_split():
    d = _rand_dense(200, 64, 0.2, 5)
    d[:20] = torch.randn(20, 64)  # heavy head
    v, ri, ro, ci = U.dense_to_sparse(d)
    for parts in (1, 2, 3, 8):
        ranges = U.nnz_balanced_row_split(ro, parts)
        assert ranges[0][0] == 0 and ranges[-1][1] == 200
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(parts - 1))
        sizes = [int(ro[e] - ro[b]) for b, e in ranges]
        assert sum(sizes) == int(ro[-1])
        assert max(sizes) <= int(ro[-1]) / parts + 64  # within one row of the ideal cut
    b, e = U.nnz_balanced_row_split(ro, 4)[2]
    sv, sri, sro, sci = U.slice_csr_rows(v, ro, ci, b, e)
    assert torch.equal(U.sparse_to_dense(sv, sro, sci, e - b, 64), d[b:e])
    empty = torch.zeros(5, dtype=torch.int32)
    assert U.nnz_balanced_row_split(empty, 2) == [(0, 0), (0, 4)] or U.nnz_balanced_row_split(empty, 2)[-1][1] == 4


def test_oracle_dense_to_csr_agrees_with_host_helper():
    """The numpy oracle of the dense -> CSR conversion and the torch host helper agree."""
    import numpy as np
    import torch
    from intrasm_engine_b200.pytorch.utils import dense_to_sparse
    from oracle import oracle
    rng = np.random.default_rng(3)
    a = rng.standard_normal((37, 53)).astype(np.float32)
    a[rng.random(a.shape) > 0.2] = 0
    a[5] = a[20]
    a[9] = 0
    v, ri, ro, ci = oracle.dense_to_csr(a)
    tv, tri, tro, tci = dense_to_sparse(torch.as_tensor(a))
    assert np.array_equal(v, tv.numpy()) and np.array_equal(ri, tri.numpy())
    assert np.array_equal(ro, tro.numpy()) and np.array_equal(ci, tci.numpy())
    rv, _, rro, rci = oracle.dense_to_csr(a, relu=True)
    assert np.all(rv > 0) and rro[-1] == (a > 0).sum() and len(rci) == len(rv)
