"""Partitioning of the path over GPUs (one process per GPU).

Encode (Viterbi, LDLQ): tiles and W rows are independent, so rank r of G takes a contiguous run of 16-row tile rows
and no data crosses GPUs. Decode (GEMV/GEMM): rotated-row tensor parallelism as the reference's Weight::load
(runtime/cuda/tensor_model.cpp:105-124): contiguous 32-row block-rows of the kernel-layout trellis per rank, the input
transform computed on every rank, the rotated products z all-gathered, the output transform on every rank.
"""


def tile_row_range(tile_rows, rank, world):
    """[begin, end) of the 16-row tile rows owned by `rank`; remainders go to the lowest ranks."""
    base, extra = divmod(tile_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def block_row_range(n_out, rank, world):
    """[row0, row0 + rows) of the output rows owned by `rank`, in whole 32-row block-rows, equal on every rank (the
    all-gather needs equal counts): n_out must be a multiple of 32 * world."""
    if n_out % (32 * world):
        raise ValueError("out = %d is not a multiple of 32 x %d ranks" % (n_out, world))
    rows = n_out // world
    return rank * rows, rows
