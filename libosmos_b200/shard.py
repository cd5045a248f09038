"""Dense projections across GPUs: a matrix's output rows split among the ranks, no collective on the data path.

A row's sum lives on one GPU and is the same arithmetic whatever the split, so a rank's slice of y has the bits of the
whole product's - the reference's kernels have the same property (a row is a block's, kernels/mv.h:14-70,
kernels/mmq.hip:60-151), which is what makes the split free. Slices are whole tiles of 128 rows (the tensor-core
kernels' row tile), the first ranks taking the remainder.
"""
ROW_TILE = 128


def row_range(rank, world, rows, tile=ROW_TILE):
    """rows [r0, r1) of a `rows`-row matrix that `rank` of `world` computes; rows in whole tiles"""
    if rows % tile:
        raise ValueError("%d rows are not whole tiles of %d" % (rows, tile))
    tiles = rows // tile
    per, rem = divmod(tiles, world)
    first = rank * per + min(rank, rem)
    return first * tile, (first + per + (1 if rank < rem else 0)) * tile


class DenseRows:
    """A rank's slice of one Q4_K matrix and the prefill step on it: the tokens' rows to int8 (every rank does all the
    tokens: the activations are not split), then mmq_group over the slice's rows into this rank's columns of y."""

    def __init__(self, lib, dev, type_id, rows, cols, host_matrix, rank=0, world=1, copies=1, max_tok=512):
        import torch
        from . import synth
        self.lib, self.dev, self.tid, self.cols = lib, dev, type_id, cols
        self.r0, self.r1 = row_range(rank, world, rows)
        self.rows = self.r1 - self.r0
        rb = synth.tensor_bytes(type_id, 1, cols)
        part = host_matrix.reshape(rows, rb)[self.r0:self.r1].reshape(-1)
        self.nb = int(part.size)
        self.pool = torch.from_numpy(part.copy()).to(dev).repeat(copies) if self.rows else None
        self.copies = copies
        n16 = (max_tok + 15) // 16 * 16
        self.x8 = torch.zeros(n16 * cols, dtype=torch.int8, device=dev)
        self.dx = torch.zeros(n16 * cols // 32, dtype=torch.float32, device=dev)
        self.sx = torch.zeros_like(self.dx)
        self.idx = torch.arange(max_tok, dtype=torch.int32, device=dev)
        self.zero = torch.zeros(1, dtype=torch.int32, device=dev)
        self.cnt = torch.zeros(1, dtype=torch.int32, device=dev)
        self._cnt = 0  # (what the device word holds)
        self.tabs = [torch.tensor([self.pool.data_ptr() + c * self.nb], dtype=torch.int64, device=dev) for c in range(copies)] if self.rows else []

    def step(self, x, n_tok, y, copy, stream):
        """x [n_tok, cols] F32 on the device -> y [n_tok, this rank's rows] F32 (row stride: the slice's rows)"""
        lib = self.lib
        if not lib.mmq_x8_rows(x.data_ptr(), self.cols, self.idx.data_ptr(), n_tok, self.cols, self.x8.data_ptr(),
                               self.dx.data_ptr(), self.sx.data_ptr(), stream):
            raise RuntimeError("libosmos_b200 refused mmq_x8_rows")
        if not self.rows:
            return
        if n_tok != self._cnt:
            self.cnt.fill_(n_tok)
            self._cnt = n_tok
        if not lib.mmq_group(self.tid, self.tabs[copy % self.copies].data_ptr(), self.cnt.data_ptr(), 1, n_tok, self.rows,
                             self.cols, self.x8.data_ptr(), self.dx.data_ptr(), self.sx.data_ptr(), self.zero.data_ptr(),
                             y.data_ptr(), self.zero.data_ptr(), self.rows, stream):
            raise RuntimeError("libosmos_b200 refused mmq_group")
