"""World-size-2 checks of the sharding logic on CPU (gloo).  The GEMM itself is replaced
by the CPU oracle here — these tests cover who owns which rows/columns, the K-chunk
accumulation order and the all-gather layout, not the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from axiom_b200.multi_gpu import ColumnShardedMLP, RowShardedMLP, gathered_to_full, shard_bounds


class OracleEngine:
    """Same call signature as axiom_b200.engine.Engine.gemm_bias_act, computed by the C oracle on CPU tensors."""

    def __init__(self):
        from oracle_lib import Oracle
        self.o = Oracle()

    def gemm_bias_act(self, A, B, bias, out, M, N, K, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, act="none"):
        a = np.ascontiguousarray(A.numpy()[:M, :K])
        b = np.ascontiguousarray(B.numpy()[:K, :N])
        c = alpha * self.o.gemm(a, b)
        if beta != 0.0:
            c = c + beta * out.numpy()
        c = self.o.bias_act(np.ascontiguousarray(c, dtype=np.float32), None if bias is None else bias.numpy(), act)
        out.copy_(torch.from_numpy(c))
        return out


def _mlp_inputs():
    from oracle_lib import Oracle
    o = Oracle()
    dims = [48, 64, 96, 32]
    x = o.uniform((20, dims[0]), 3)
    Ws = [o.normal((dims[i], dims[i + 1]), 10 + i, sigma=1.0 / np.sqrt(dims[i])) for i in range(3)]
    bs = [o.uniform((dims[i + 1],), 20 + i) for i in range(3)]
    h = x
    for W, b in zip(Ws, bs):
        h = o.bias_act(o.gemm(h, W), b, "gelu")
    return x, Ws, bs, h


def test_shard_bounds_cover_everything():
    for n in (0, 1, 7, 8, 1000):
        for world in (1, 2, 3, 8):
            parts = [shard_bounds(n, world, r) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, Ws, bs, want = _mlp_inputs()
        eng = OracleEngine()
        new_empty = lambda shape: torch.empty(shape, dtype=torch.float32)
        # rows
        r0, r1 = shard_bounds(x.shape[0], world, rank)
        y_rows = RowShardedMLP(eng, [torch.from_numpy(W) for W in Ws], [torch.from_numpy(b) for b in bs]).forward(
            torch.from_numpy(np.ascontiguousarray(x[r0:r1])), new_empty)
        np.testing.assert_allclose(y_rows.numpy(), want[r0:r1], atol=1e-5)
        # columns + all-gather
        slabs, bias_slabs = [], []
        for W, b in zip(Ws, bs):
            c0, c1 = shard_bounds(W.shape[1], world, rank)
            slabs.append(torch.from_numpy(np.ascontiguousarray(W[:, c0:c1])))
            bias_slabs.append(torch.from_numpy(np.ascontiguousarray(b[c0:c1])))
        ag = lambda dst, src: dist.all_gather_into_tensor(dst.view(-1, dst.shape[-1]), src)
        y = ColumnShardedMLP(eng, slabs, bias_slabs, world, rank, ag).forward(torch.from_numpy(x), new_empty)
        np.testing.assert_allclose(gathered_to_full(y).numpy(), want, atol=1e-5)
        results[rank] = "ok"
    except Exception as exc:  # surfaced by the parent
        results[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


def test_row_and_column_sharded_mlp_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}
