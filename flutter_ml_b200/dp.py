"""Host-side plumbing of the data-parallel step: which rows a rank owns and how the NCCL unique id
reaches every rank.  The exchange itself is `fml_dp_allreduce_sum` (NCCL over NVLink) on the flat
gradient arena; the reference has no multi-device code."""
from __future__ import annotations

from typing import Callable, Tuple


def shard_rows(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open row range of `rank` when `n_rows` samples are split over `world` ranks; the first
    `n_rows % world` ranks take one extra row, so every sample is owned exactly once."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def broadcast_unique_id(dist, make_id: Callable[[], bytes], device="cpu") -> bytes:
    """Rank 0 creates the 128-byte id, every rank returns the same bytes.  `dist` is an initialised
    torch.distributed module (any backend)."""
    import torch
    buf = torch.zeros(128, dtype=torch.uint8, device=device)
    if dist.get_rank() == 0:
        raw = make_id()
        if len(raw) != 128:
            raise ValueError("the unique id must be 128 bytes")
        buf.copy_(torch.tensor(list(raw), dtype=torch.uint8))
    dist.broadcast(buf, src=0)
    return bytes(buf.cpu().tolist())


def init_data_parallel(ctx, dist, rank: int, world: int, device="cpu", max_ctas: int = 0):
    """Create the NCCL communicator of `ctx` (no-op for a single rank).  `max_ctas` > 0 limits the SMs a collective
    occupies, for exchanges that run beside persistent kernels (see Context.set_sm_reserve)."""
    import ctypes
    if max_ctas:
        ctx.check(ctx.lib.fml_dp_set_max_ctas(ctx.h, int(max_ctas)))
    if world == 1:
        ctx.check(ctx.lib.fml_dp_init(ctx.h, bytes(128), 0, 1))
        return

    def make():
        raw = ctypes.create_string_buffer(128)
        rc = ctx.lib.fml_dp_unique_id(raw)
        if rc != 0:
            raise RuntimeError(ctx.lib.fml_last_error(None).decode())
        return raw.raw
    uid = broadcast_unique_id(dist, make, device)
    ctx.check(ctx.lib.fml_dp_init(ctx.h, uid, rank, world))
