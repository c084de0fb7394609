"""N-sharded / K-sharded partition logic on CPU: two gloo ranks, with the C oracle as the per-rank GEMM
(the product's per-rank GEMM is the CUDA kernel; only the partitioning and the collective are under
test here)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_dot(a, b, out=None, out_dtype=None, row_scale=None, col_scale=None, alpha=1.0, **_):
    r = a.float() @ b.float() * alpha
    if row_scale is not None:
        r = r * row_scale[:, None]
    if col_scale is not None:
        r = r * col_scale[None, :]
    r = r.to(out_dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from triton_ext_b200 import parallel as par
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(4)
        m, n, k = 64, 96, 160
        a = torch.randn(m, k, generator=g).bfloat16()
        b = (torch.randn(k, n, generator=g) * 0.02).bfloat16()
        rs = torch.rand(m, generator=g) + 0.5
        cs = torch.rand(n, generator=g) + 0.5
        full = _oracle_dot(a, b, out_dtype=torch.bfloat16, row_scale=rs, col_scale=cs)
        # N-sharded: panels are independent, reassembly is a concatenation
        n0, n1 = par.split_range(n, world, rank, align=16)
        panel = par.n_sharded_dot(a, b[:, n0:n1], out_dtype=torch.bfloat16, row_scale=rs, col_scale_shard=cs[n0:n1],
                                  local_dot=_oracle_dot)
        ok_n = torch.equal(panel.view(torch.int16), full[:, n0:n1].contiguous().view(torch.int16))
        # K-sharded: fp32 partials, reduce-scatter along M
        k0, k1 = par.split_range(k, world, rank, align=32)
        for chunks in (1, 2):
            rows = par.k_sharded_dot(a[:, k0:k1], b[k0:k1, :], out_dtype=torch.bfloat16, row_scale=rs, col_scale=cs,
                                     local_dot=_oracle_dot, chunks=chunks)
            m0 = rank * (m // world)
            want = full[m0:m0 + m // world]
            ok_k = bool(((rows.float() - want.float()).abs() <= 1e-2 + 1e-2 * want.float().abs()).all())
            q.put((rank, chunks, ok_n, ok_k, tuple(rows.shape)))
    finally:
        dist.destroy_process_group()


def test_split_range():
    from triton_ext_b200 import parallel as par
    assert [par.split_range(28672, 8, r, 256) for r in range(8)] == [(r * 3584, (r + 1) * 3584) for r in range(8)]
    parts = [par.split_range(100, 3, r, 16) for r in range(3)]
    assert parts[0][0] == 0 and parts[-1][1] == 100
    assert all(parts[i][1] == parts[i + 1][0] for i in range(2))
    assert all(lo % 16 == 0 for lo, _ in parts)
    with pytest.raises(ValueError):
        par.split_range(10, 2, 2)


def test_two_rank_partitions_match_unsharded():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(120) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    results = [q.get(timeout=5) for _ in range(world * 2)]
    assert len(results) == 4
    for rank, chunks, ok_n, ok_k, shape in results:
        assert ok_n and ok_k, (rank, chunks)
        assert shape == (32, 96)
