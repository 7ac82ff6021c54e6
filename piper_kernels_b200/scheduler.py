"""Host scheduler: shard the flattened (batch x heads) axis across the GPUs of one box.

Every (batch, head) of an attention call is independent (its softmax, K mean, V mean / scale
and key order are all per head), so the path needs no collective: each rank runs the prepass
and the fused kernel on a contiguous chunk of flat heads and keeps its slice of the output.
Outputs are gathered only when a caller asks for the whole tensor (for reporting).
"""

from __future__ import annotations

import torch


def shard_heads(flat_heads: int, world: int, rank: int) -> range:
    """Contiguous, balanced chunk of ``range(flat_heads)`` owned by ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(flat_heads, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def sharded_attention(op, query, key, value, *, world: int, rank: int, **kwargs) -> tuple[torch.Tensor, range]:
    """Run ``op`` (``piper_attention`` / ``sage_attention_2pp`` or any function with their
    signature) on this rank's heads.  Inputs are full ``[B,H,S,D]`` tensors (or views of
    them); returns the output slice ``[1, n_local, Sq, D]`` and the flat-head range."""
    b, h = query.shape[:2]
    mine = shard_heads(b * h, world, rank)
    flat = lambda t: t.reshape(b * h, *t.shape[2:]) if t.is_contiguous() else t.flatten(0, 1)  # noqa: E731
    if len(mine) == 0:
        return query.new_empty((1, 0, query.shape[2], query.shape[3])), mine
    sl = slice(mine.start, mine.stop)
    out = op(flat(query)[sl].unsqueeze(0), flat(key)[sl].unsqueeze(0), flat(value)[sl].unsqueeze(0), **kwargs)
    return out, mine


def gather_outputs(local: torch.Tensor, mine: range, flat_heads: int, shape, group=None) -> torch.Tensor | None:
    """Collect every rank's slice on rank 0 (reporting only; not part of the timed path)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    pieces = [None] * world
    dist.gather_object((mine.start, mine.stop, local.cpu()), pieces if rank == 0 else None, dst=0, group=group)
    if rank != 0:
        return None
    full = torch.empty((flat_heads, *shape[2:]), dtype=local.dtype)
    for start, stop, piece in pieces:
        if stop > start:
            full[start:stop] = piece[0]
    return full.reshape(shape)


def attention_from_host(op, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                        out_host: torch.Tensor, device, *, heads_per_chunk: int = 8, **kwargs) -> torch.Tensor:
    """Run ``op`` on inputs that live in (pinned) host memory and write the result to host memory.

    Heads are independent, so the flat (batch x heads) axis is cut into chunks; the upload of
    chunk i+1, the compute of chunk i and the download of chunk i-1 overlap on three CUDA
    streams.  ``q_host``/``k_host``/``v_host`` are ``[B,H,S,D]`` (``k_host``/``v_host`` may be
    strided views of one buffer); ``out_host`` is a contiguous ``[B,H,Sq,D]`` host tensor.
    Returns ``out_host`` after synchronising the three streams.
    """
    device = torch.device(device)
    b, h = q_host.shape[:2]
    flat = b * h
    fq, fk, fv = (t.flatten(0, 1) for t in (q_host, k_host, v_host))
    fo = out_host.view(flat, *out_host.shape[2:])
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    main = torch.cuda.current_stream(device)
    up.wait_stream(main)
    down.wait_stream(main)
    pending = None
    for start in range(0, flat, heads_per_chunk):
        sl = slice(start, min(flat, start + heads_per_chunk))
        with torch.cuda.stream(up):
            dq, dk, dv = (t[sl].to(device, non_blocking=True).unsqueeze(0) for t in (fq, fk, fv))
            uploaded = torch.cuda.Event()
            uploaded.record(up)
        main.wait_event(uploaded)
        for t in (dq, dk, dv):
            t.record_stream(main)
        out = op(dq, dk, dv, **kwargs)
        computed = torch.cuda.Event()
        computed.record(main)
        with torch.cuda.stream(down):
            down.wait_event(computed)
            out.record_stream(down)
            fo[sl].copy_(out[0], non_blocking=True)
        pending = (dq, dk, dv, out)
    del pending
    main.wait_stream(down)
    main.wait_stream(up)
    return out_host
