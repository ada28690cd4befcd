"""Sharding of large GEMMs and of a chained MLP over the GPUs of one box.

One process per GPU (torch.distributed).  Two partitions are offered:

* rows (M): every rank owns M/g rows of the input and of every activation; weights
  are replicated.  No data-path collective at all.
* columns (N): every rank owns N_l/g output columns of every layer (weights and
  biases sliced by column), computes its slab with the bias + activation fused in
  the GEMM epilogue, and ONE all-gather per layer makes the full activation
  available to every rank for the next layer.  The gather lands in a
  ``[g][M][N_l/g]`` buffer — each rank's slab contiguous, so the collective is a
  plain contiguous all-gather — and the next layer reads that buffer in place as
  its [M, N_l] operand (the operand-split pre-pass walks the g chunks), so no
  re-layout pass and no accumulating calls are needed.

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

    def __init__(self, engine, weights, biases, act="gelu", prepare=False):
        """prepare: keep every weight's tensor-core operand planes (axb_weight_prepare) so a forward pass splits
        activations only; the weights must then stay unchanged until close()."""
        assert len(weights) == len(biases)
        self.engine, self.weights, self.biases, self.act = engine, list(weights), list(biases), act
        self.prepared = [engine.weight_prepare(W) for W in self.weights] if prepare else None

    def forward(self, x_rows, new_empty):
        h = x_rows
        for l, (W, b) in enumerate(zip(self.weights, self.biases)):
            M, K = h.shape
            N = W.shape[1]
            out = new_empty((M, N))
            if self.prepared is not None:
                self.engine.gemm_prepared(h, self.prepared[l], b, out, M, act=self.act)
            else:
                self.engine.gemm_bias_act(h, W, b, out, M, N, K, act=self.act)
            h = out
        return h

    def close(self):
        for w in self.prepared or []:
            self.engine.weight_release(w)
        self.prepared = None


class ColumnShardedMLP:
    """The same chain with every layer's output columns split over the ranks and one all-gather per layer."""

    def __init__(self, engine, weight_slabs, bias_slabs, world, rank, all_gather, act="gelu", prepare=False):
        """weight_slabs[l]: this rank's [K_l, N_l/g] column slab of layer l (contiguous); bias_slabs[l]: [N_l/g].
        all_gather(dst[g, M, n], src[M, n]) performs the collective (torch.distributed.all_gather_into_tensor).
        prepare: keep every slab's tensor-core operand planes (the slabs must then stay unchanged until close())."""
        self.engine, self.world, self.rank, self.act = engine, world, rank, act
        self.weight_slabs, self.bias_slabs, self.all_gather = list(weight_slabs), list(bias_slabs), all_gather
        self.prepared = [engine.weight_prepare(W) for W in self.weight_slabs] if prepare else None

    def close(self):
        for w in self.prepared or []:
            self.engine.weight_release(w)
        self.prepared = None

    def forward(self, x_full, new_empty):
        """x_full: the full [M, K_0] input on every rank.  Returns the gathered [g, M, N_last/g] output."""
        g = self.world
        gathered = None
        for l, (W, b) in enumerate(zip(self.weight_slabs, self.bias_slabs)):
            n = W.shape[1]
            if gathered is None:
                M, K = x_full.shape
                slab = new_empty((M, n))
                if self.prepared is not None:
                    self.engine.gemm_prepared(x_full, self.prepared[l], b, slab, M, act=self.act)
                else:
                    self.engine.gemm_bias_act(x_full, W, b, slab, M, n, K, act=self.act)
            else:
                # the previous layer's gather buffer [g][M][k] is read in place as the [M, g*k] operand
                _, M, kc = gathered.shape
                slab = new_empty((M, n))
                if self.prepared is not None:
                    self.engine.gemm_prepared_scatter(gathered, g, kc, self.prepared[l], b, slab, [], M, act=self.act)
                elif hasattr(self.engine, "gemm_gathered_scatter"):
                    self.engine.gemm_gathered_scatter(gathered, g, kc, W, b, slab, [], M, n, act=self.act)
                else:   # engines without the gathered-operand entry: g accumulating calls over the K-chunks
                    for c in range(g):
                        last = c == g - 1
                        self.engine.gemm_bias_act(gathered[c], W[c * kc:(c + 1) * kc], b if last else None, slab, M, n, kc,
                                                  beta=0.0 if c == 0 else 1.0, act=self.act if last else "none")
            gathered = new_empty((g, slab.shape[0], n))
            self.all_gather(gathered, slab)
        return gathered


def gathered_to_full(gathered):
    """[g, M, n] -> [M, g*n] (a copy; for checking results, not part of the data path)."""
    g, M, n = gathered.shape
    return gathered.permute(1, 0, 2).reshape(M, g * n)


class PeerScatterColumnMLP:
    """Column-sharded MLP whose GEMM epilogue does the all-gather: the last accumulating call of a layer
    stores this rank's finished slab straight into EVERY rank's ``[g][M][n]`` gather buffer (peer stores
    over NVLink from the tensor-core kernel's epilogue, ``axb_gemm_bias_act_scatter``), so the transfer
    overlaps the MMAs tile by tile and no separate collective moves data.  One tiny all-reduce per layer
    orders the peers' reads after everybody's stores.

    Gather buffers are plain device allocations (``axb_storage_alloc``) shared through CUDA IPC handles that
    the ranks exchange once with ``all_gather_object``; they are reused every step (a rank can only start
    the next step after the last layer's synchronisation, by which time every rank has finished reading the
    buffers of all layers but the last; with a single layer the caller must not start the next step before
    its peers have consumed the output, e.g. by a barrier of its own)."""

    def __init__(self, engine, weight_slabs, bias_slabs, world, rank, batch, dist, act="gelu", prepare=False):
        import torch
        self.engine, self.world, self.rank, self.act, self.dist = engine, world, rank, act, dist
        self.weight_slabs, self.bias_slabs, self.batch = list(weight_slabs), list(bias_slabs), batch
        # prepare: the slabs' operand planes are made once (the slabs must then stay unchanged until close())
        self.prepared = [engine.weight_prepare(W) for W in self.weight_slabs] if prepare else None
        self._token = torch.zeros(1, device="cuda")
        self.local, self.peers, self._opened = [], [], []
        for W in self.weight_slabs:
            n = W.shape[1]
            nbytes = world * batch * n * 4
            ptr = engine.storage_alloc(nbytes)
            handles = [None] * world
            dist.all_gather_object(handles, engine.ipc_get_handle(ptr))
            ptrs = []
            for r, h in enumerate(handles):
                if r == rank:
                    ptrs.append(ptr)
                else:
                    q = engine.ipc_open_handle(h)
                    self._opened.append(q)
                    ptrs.append(q)
            self.local.append(ptr)
            self.peers.append(ptrs)
        dist.barrier()

    def forward(self, x_full, new_empty):
        """x_full: the full [M, K_0] input on every rank; returns the device pointer of the gathered
        [g, M, n_last] output in this rank's memory and n_last."""
        g, M = self.world, self.batch
        n, prev_n = 0, 0
        for l, (W, b) in enumerate(zip(self.weight_slabs, self.bias_slabs)):
            n = W.shape[1]
            slab = new_empty((M, n))
            # every rank's gather buffer, at the slab this rank owns
            dests = [p + self.rank * M * n * 4 for p in self.peers[l]]
            if self.prepared is not None:
                src, chunks, kc = (x_full, 0, 0) if l == 0 else (self.local[l - 1], g, prev_n)
                self.engine.gemm_prepared_scatter(src, chunks, kc, self.prepared[l], b, slab, dests, M, act=self.act)
            elif l == 0:
                self.engine.gemm_bias_act_scatter(x_full, W, b, slab, dests, M, n, x_full.shape[1], act=self.act)
            else:
                self.engine.gemm_gathered_scatter(self.local[l - 1], g, prev_n, W, b, slab, dests, M, n, act=self.act)
            self._exchange_token()                      # everybody's stores are done before anybody reads
            prev_n = n
        return self.local[-1], n

    def _exchange_token(self):
        """The all-reduce runs on torch's current stream, the GEMMs on the engine's: order the collective after this
        rank's stores and the next layer's reads after the collective, whichever streams those are."""
        import torch
        cur = torch.cuda.current_stream()
        sp = getattr(self.engine, "stream_ptr", 0)
        eng_stream = torch.cuda.ExternalStream(sp) if sp else torch.cuda.default_stream()
        same = eng_stream.cuda_stream == cur.cuda_stream
        if not same:
            cur.wait_stream(eng_stream)
        self.dist.all_reduce(self._token)
        if not same:
            eng_stream.wait_stream(cur)

    def close(self):
        for w in self.prepared or []:
            self.engine.weight_release(w)
        self.prepared = None
        self.dist.barrier()
        for q in self._opened:
            self.engine.ipc_close_handle(q)
        self.dist.barrier()
        for p in self.local:
            self.engine.storage_free(p)
        self._opened, self.local = [], []
