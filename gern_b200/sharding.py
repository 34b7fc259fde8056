"""Row sharding of the fused kernels across the GPUs of one box (one process per GPU).

The reference is single-GPU (no cudaSetDevice, stream or collective anywhere in its tree), so this
layer has no counterpart there; it follows the partitioning the kernels allow:

  * matrix multiply : M panels of A and C per rank, B replicated       -> no exchange
  * row softmax     : contiguous row blocks                            -> no exchange
  * GEMM->softmax->GEMM chain: Q / O row blocks, K and V replicated    -> no exchange
  * fused blur      : bands of output rows; a band needs the first two input rows of the next
                      band (the 2-row halo of the 3-tap vertical pass)  -> one neighbour exchange

Only index arithmetic and the halo exchange live here; compute goes through the C ABI.
"""
from __future__ import annotations

from dataclasses import dataclass


def row_block(total_rows: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of the contiguous row block of `rank` (blocks differ by at most one row)."""
    base, extra = divmod(total_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


@dataclass(frozen=True)
class BlurBand:
    """What one rank holds and produces for an image of in_rows x in_cols sharded by rows."""
    rank: int
    world: int
    in_begin: int      # first input row this rank owns
    in_end: int        # one past the last input row this rank owns
    out_begin: int     # first output row this rank produces (== in_begin)
    out_end: int       # one past the last output row this rank produces
    halo_rows: int     # rows needed from the next rank (2, or 0 for the last non-empty band)

    @property
    def band_rows(self) -> int:
        return self.in_end - self.in_begin

    @property
    def out_rows(self) -> int:
        return self.out_end - self.out_begin

    @property
    def sends_halo(self) -> bool:
        """True if the previous rank needs this rank's first two rows."""
        return self.rank > 0 and self.band_rows > 0

    @property
    def recvs_halo(self) -> bool:
        return self.halo_rows > 0


def blur_band(in_rows: int, world: int, rank: int) -> BlurBand:
    """Input rows are dealt in contiguous blocks; rank r produces the output rows whose first
    input row it owns.  Output row i reads input rows i, i+1, i+2, so every band but the last
    reads two rows of its successor.  Bands must hold at least 2 rows (or be the only one)."""
    begin, end = row_block(in_rows, world, rank)
    out_total = max(in_rows - 2, 0)
    if world > 1 and in_rows // world < 2:
        raise ValueError(f"{in_rows} rows cannot be sharded {world} ways with a 2-row halo")
    out_begin = min(begin, out_total)
    out_end = min(end, out_total)
    halo = 2 if (rank < world - 1 and out_end > out_begin) else 0
    return BlurBand(rank, world, begin, end, out_begin, out_end, halo)


def exchange_blur_halo(dist, band: BlurBand, own_first_rows, halo_buffer):
    """Posts the neighbour exchange of one step: send this rank's first two rows to rank-1,
    receive the next rank's first two rows into `halo_buffer`.  Returns the request list
    (torch.distributed work handles) for the caller to wait on, on the stream or thread it likes.
    Works with any backend (NCCL over NVLink on GPUs, gloo on CPU)."""
    ops = []
    if band.sends_halo:
        ops.append(dist.P2POp(dist.isend, own_first_rows, band.rank - 1))
    if band.recvs_halo:
        ops.append(dist.P2POp(dist.irecv, halo_buffer, band.rank + 1))
    return dist.batch_isend_irecv(ops) if ops else []
