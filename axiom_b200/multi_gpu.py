"""Sharding of large GEMMs and of a chained MLP over the GPUs of one box.

One process per GPU (torch.distributed).  Two partitions are offered:

* rows (M): every rank owns M/g rows of the input and of every activation; weights
  are replicated.  No data-path collective at all.
* columns (N): every rank owns N_l/g output columns of every layer (weights and
  biases sliced by column), computes its slab with the bias + activation fused in
  the GEMM epilogue, and ONE all-gather per layer makes the full activation
  available to every rank for the next layer.  The gather lands in a
  ``[g][M][N_l/g]`` buffer — each rank's slab contiguous, so the collective is a
  plain contiguous all-gather — and the next layer consumes that buffer as g
  chunks of its K dimension (g accumulating GEMM calls, bias + activation on
  the last), so no re-layout pass is needed.

The reference is single-device: this module has no counterpart there.  The
GEMMs are always the engine's kernels; ``torch`` only owns buffers and the
process group.
"""
from __future__ import annotations


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the contiguous shard `rank` of `n` items over `world` ranks (sizes differ by at most one)."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


class RowShardedMLP:
    """y = act(...act(x W1 + b1)... Wn + bn) on this rank's rows of x; weights replicated, no communication."""

    def __init__(self, engine, weights, biases, act="gelu"):
        assert len(weights) == len(biases)
        self.engine, self.weights, self.biases, self.act = engine, list(weights), list(biases), act

    def forward(self, x_rows, new_empty):
        h = x_rows
        for W, b in zip(self.weights, self.biases):
            M, K = h.shape
            N = W.shape[1]
            out = new_empty((M, N))
            self.engine.gemm_bias_act(h, W, b, out, M, N, K, act=self.act)
            h = out
        return h


class ColumnShardedMLP:
    """The same chain with every layer's output columns split over the ranks and one all-gather per layer."""

    def __init__(self, engine, weight_slabs, bias_slabs, world, rank, all_gather, act="gelu"):
        """weight_slabs[l]: this rank's [K_l, N_l/g] column slab of layer l (contiguous); bias_slabs[l]: [N_l/g].
        all_gather(dst[g, M, n], src[M, n]) performs the collective (torch.distributed.all_gather_into_tensor)."""
        self.engine, self.world, self.rank, self.act = engine, world, rank, act
        self.weight_slabs, self.bias_slabs, self.all_gather = list(weight_slabs), list(bias_slabs), all_gather

    def forward(self, x_full, new_empty):
        """x_full: the full [M, K_0] input on every rank.  Returns the gathered [g, M, N_last/g] output."""
        g = self.world
        chunks = [x_full]                     # the current layer's input as a list of K-chunks [M, k_c]
        gathered = None
        for W, b in zip(self.weight_slabs, self.bias_slabs):
            M = chunks[0].shape[0]
            n = W.shape[1]
            slab = new_empty((M, n))
            k0 = 0
            for c, xc in enumerate(chunks):
                kc = xc.shape[1]
                last = c == len(chunks) - 1
                # rows k0 .. k0+kc of this rank's weight slab (a contiguous block of rows)
                self.engine.gemm_bias_act(xc, W[k0:k0 + kc], b if last else None, slab, M, n, kc,
                                          beta=0.0 if c == 0 else 1.0, act=self.act if last else "none")
                k0 += kc
            assert k0 == W.shape[0]
            gathered = new_empty((g, M, n))
            self.all_gather(gathered, slab)
            chunks = [gathered[r] for r in range(g)]
        return gathered


def gathered_to_full(gathered):
    """[g, M, n] -> [M, g*n] (a copy; for checking results, not part of the data path)."""
    g, M, n = gathered.shape
    return gathered.permute(1, 0, 2).reshape(M, g * n)
