"""Multi-GPU partitioning of the kernel set: one process per GPU over `torch.distributed`.

The reference is single-device.  Every kernel of the set shards over independent units, so no kernel
ever reads another GPU's memory:

  softmax / LayerNorm / RMSNorm / row cumsum   contiguous row blocks          no collective
  GELU / add                                   contiguous element ranges      no collective
  matmul                                       M-blocks of A and C (B, bias replicated)   no collective
  attention                                    (batch, head) slices           no collective
  histogram                                    element ranges -> local bins   all-reduce(sum) of int32 bins
  flat cumsum                                  contiguous shard per rank      all-gather of one total per rank:
                                               local total -> exclusive offset -> local scan seeded with it

The two collectives move at most 16 KB (4096 int32 bins) or world_size scalars, so they are
latency-bound NCCL calls on the launch stream.  The helpers take the local compute as callables, which
lets the same logic run among CPU ranks over gloo in the tests.
"""

from __future__ import annotations

from typing import Any, Callable

import numpy as np


def shard_range(n: int, rank: int, world: int, align: int = 1) -> tuple[int, int]:
    """[start, stop) of rank's contiguous share of `n` units; shares differ by at most `align` units
    and every boundary except the last is a multiple of `align`."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a group of {world}")
    blocks = -(-n // align)
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * align, n), min(b1 * align, n)


def exclusive_offsets(totals: np.ndarray) -> np.ndarray:
    """Exclusive prefix of per-rank totals in the totals' own arithmetic.

    int32/uint32 totals wrap modulo 2**32 (added as uint32, as the scan kernel does); float32 totals
    are added in float32, rank by rank.
    """
    t = np.asarray(totals)
    if t.dtype.kind in "iu":
        u = t.astype(np.uint32) if t.dtype.itemsize == 4 else t.astype(np.uint64)
        ex = np.concatenate([np.zeros(1, u.dtype), np.cumsum(u[:-1], dtype=u.dtype)])
        return ex.view(t.dtype) if t.dtype.itemsize == u.dtype.itemsize else ex.astype(t.dtype)
    out = np.zeros_like(t)
    acc = t.dtype.type(0)
    for i in range(len(t)):
        out[i] = acc
        acc = t.dtype.type(acc + t[i])
    return out


def allreduce_histogram(hist: Any, group: Any = None) -> Any:
    """Sums per-rank int32 bin counts in place across the group (NCCL on GPU tensors, gloo on CPU)."""
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(hist, op=dist.ReduceOp.SUM, group=group)
    return hist


def sharded_histogram(x_local: Any, num_bins: int, lo: float, hi: float, local_histogram: Callable,
                      group: Any = None) -> Any:
    """Histogram of an array split across ranks: local counts, then one all-reduce of the bins."""
    return allreduce_histogram(local_histogram(x_local, num_bins, lo, hi), group)


def host_offset(gathered: Any, rank: int) -> Any:
    """Exclusive offset of `rank` from the gathered totals, computed on the host (CPU ranks over gloo)."""
    import torch

    offs = exclusive_offsets(gathered.cpu().numpy())
    return torch.from_numpy(offs[rank : rank + 1].copy()).to(gathered.device)


def sharded_cumsum(x_local: Any, local_total: Callable[[Any], Any], local_scan: Callable[[Any, Any], Any],
                   group: Any = None, offset: Callable[[Any, int], Any] | None = None) -> Any:
    """Inclusive scan of one flat array split contiguously across ranks (rank r holds shard r).

    `local_total(x_local)` returns a one-element torch tensor (accumulator dtype) with the shard's sum;
    `local_scan(x_local, seed)` returns the shard's inclusive scan with `seed` (a one-element tensor,
    the exclusive offset) added; `offset(gathered, rank)` turns the all-gathered totals into that seed
    (default: `cuda_offset` for CUDA tensors, which is a one-thread kernel on the launch stream, so the
    two passes and the all-gather between them stay stream-ordered with no host round trip; `host_offset`
    otherwise).  Traffic per rank: the shard is read twice and written once.
    """
    import torch
    import torch.distributed as dist

    total = local_total(x_local)
    if not (dist.is_initialized() and dist.get_world_size(group) > 1):
        return local_scan(x_local, torch.zeros_like(total))
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    gathered = torch.empty(world, dtype=total.dtype, device=total.device)
    dist.all_gather_into_tensor(gathered, total.reshape(1), group=group)
    if offset is None:
        offset = cuda_offset if gathered.is_cuda else host_offset
    return local_scan(x_local, offset(gathered, rank))


# ---- CUDA-backed local steps -------------------------------------------------------------------
def cuda_total(x: Any) -> Any:
    """Shard total in the scan's accumulator type (int32 wrap / float32) as a one-element tensor."""
    import torch

    from enceladus_b200 import _native as N
    from enceladus_b200.runtime import interop

    code = interop.dtype_code(x)
    acc = torch.float32 if code in (N.F32, N.F16, N.BF16) else (torch.int64 if code == N.I64 else torch.int32)
    out = torch.empty(1, dtype=acc, device=x.device)
    N.call("enc_sum", x.data_ptr(), out.data_ptr(), x.numel(), code, interop.current_stream())
    return out


def cuda_offset(gathered: Any, rank: int) -> Any:
    """Exclusive offset of `rank` from the gathered totals, on the device and on the current stream."""
    import torch

    from enceladus_b200 import _native as N
    from enceladus_b200.runtime import interop

    code = {torch.float32: N.F32, torch.int32: N.I32, torch.int64: N.I64}[gathered.dtype]
    out = torch.empty(1, dtype=gathered.dtype, device=gathered.device)
    N.call("enc_scan_offset", gathered.data_ptr(), gathered.numel(), int(rank), out.data_ptr(), code,
           interop.current_stream())
    return out


def cuda_scan(x: Any, seed: Any) -> Any:
    """Flat inclusive scan of a device array with `seed` added to every element."""
    import torch

    from enceladus_b200 import _native as N
    from enceladus_b200.runtime import interop

    code = interop.dtype_code(x)
    out_code = N.load().enc_cumsum_out_dtype(code)
    out = torch.empty(x.numel(), dtype=torch.int32 if out_code == N.I32 else x.dtype, device=x.device)
    n = x.numel()
    N.call("enc_cumsum", x.data_ptr(), out.data_ptr(), 1, n, n, n, 0, code, seed.data_ptr(), -1,
           interop.current_stream())
    return out
