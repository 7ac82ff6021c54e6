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


class HostAttentionPipeline:
    """Attention on inputs and outputs that live in pinned host memory.

    Heads are independent, so the flat (batch x heads) axis is cut into chunks; the upload of
    chunk i+1, the compute of chunk i and the download of chunk i-1 overlap on three CUDA
    streams.  Device staging buffers (two slots per tensor) are allocated once and re-used.
    """

    def __init__(self, device, *, heads_per_chunk: int = 8):
        self.device = torch.device(device)
        self.heads_per_chunk = int(heads_per_chunk)
        self.up = torch.cuda.Stream(self.device)
        self.down = torch.cuda.Stream(self.device)
        self._slots = None
        self._key = None

    def _staging(self, q, k, v):
        key = (tuple(q.shape[2:]), tuple(k.shape[2:]), q.dtype)
        if self._key != key:
            n = self.heads_per_chunk
            mk = lambda t: torch.empty((n, *t.shape[2:]), dtype=t.dtype, device=self.device)  # noqa: E731
            self._slots = [{"q": mk(q), "k": mk(k), "v": mk(v), "out": mk(q), "free": None, "drained": None} for _ in range(2)]
            self._key = key
        return self._slots

    def __call__(self, op, q_host, k_host, v_host, out_host, **kwargs) -> torch.Tensor:
        b, h = q_host.shape[:2]
        flat = b * h
        fq, fk, fv = (t.flatten(0, 1) for t in (q_host, k_host, v_host))
        fo = out_host.view(flat, *out_host.shape[2:])
        slots = self._staging(q_host, k_host, v_host)
        main = torch.cuda.current_stream(self.device)
        self.up.wait_stream(main)
        self.down.wait_stream(main)
        for i, start in enumerate(range(0, flat, self.heads_per_chunk)):
            n = min(flat, start + self.heads_per_chunk) - start
            sl = slice(start, start + n)
            slot = slots[i % 2]
            with torch.cuda.stream(self.up):
                if slot["free"] is not None:
                    self.up.wait_event(slot["free"])  # the compute that read this slot has finished
                slot["q"][:n].copy_(fq[sl], non_blocking=True)
                slot["k"][:n].copy_(fk[sl], non_blocking=True)
                slot["v"][:n].copy_(fv[sl], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(self.up)
            main.wait_event(uploaded)
            if slot["drained"] is not None:
                main.wait_event(slot["drained"])  # the download of this slot's previous result has finished
            out = op(slot["q"][:n].unsqueeze(0), slot["k"][:n].unsqueeze(0), slot["v"][:n].unsqueeze(0), **kwargs)
            slot["out"][:n].copy_(out[0])
            slot["free"] = torch.cuda.Event()
            slot["free"].record(main)
            with torch.cuda.stream(self.down):
                self.down.wait_event(slot["free"])
                fo[sl].copy_(slot["out"][:n], non_blocking=True)
                slot["drained"] = torch.cuda.Event()
                slot["drained"].record(self.down)
        main.wait_stream(self.down)
        main.wait_stream(self.up)
        return out_host


def attention_from_host(op, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                        out_host: torch.Tensor, device, *, heads_per_chunk: int = 8, **kwargs) -> torch.Tensor:
    """One-shot form of :class:`HostAttentionPipeline` (allocates the staging buffers per call)."""
    return HostAttentionPipeline(device, heads_per_chunk=heads_per_chunk)(op, q_host, k_host, v_host, out_host, **kwargs)
