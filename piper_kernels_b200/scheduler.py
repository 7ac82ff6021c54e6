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


def plan_chunks(flat_heads: int, max_chunk: int) -> list[int]:
    """Chunk sizes (in flat heads) for the host pipeline: they ramp up 1, 1, 2, 4 ... to
    ``max_chunk`` and back down to 1, so that the first upload and the last download - the two
    transfers nothing can hide - are one head long, while the bulk moves in large chunks whose
    kernels fill whole waves of the GPU.  Every upload is at most twice the compute it hides behind."""
    flat_heads, max_chunk = int(flat_heads), max(1, int(max_chunk))
    ramp = [1]
    while ramp[-1] * 2 < max_chunk:
        ramp.append(ramp[-1] * 2)
    front = [1] + ramp if max_chunk > 1 else []
    back = ramp[::-1] if max_chunk > 1 else []
    while front or back:  # too few heads for the full ramps: shorten them from the large end
        if sum(front) + sum(back) <= flat_heads:
            break
        if len(back) >= len(front) - 1 and back:
            back.pop(0)
        else:
            front.pop()
    middle, rest = divmod(flat_heads - sum(front) - sum(back), max_chunk)
    plan = front + [max_chunk] * middle + sorted(back + ([rest] if rest else []), reverse=True)
    assert sum(plan) == flat_heads and all(0 < n <= max_chunk for n in plan)
    return plan


def suggest_heads_per_chunk(ops_per_head: float, flat_heads: int, *, target_ms: float = 0.6, tops: float = 800.0,
                            largest: int = 8) -> int:
    """Chunk size for :class:`HostAttentionPipeline`: enough heads for about half a millisecond of
    fused-kernel time (shorter chunks are bound by their dozen launches, longer ones expose more of
    the first upload and the last download and leave larger partial waves), at most ``largest`` and
    at most a quarter of the heads.  ``ops_per_head`` is 4 * q_len * kv_len * head_dim (halved for
    causal attention).  Measured per step: c4 (0.67 ms per head) 26.8 ms with 1 head, 27.0 with 2,
    27.2 with 3; c5 (0.04 ms per head) 11.8 ms with 4 heads, 13.2 with 2."""
    per_head_ms = float(ops_per_head) / (tops * 1e9)
    want = int(-(-target_ms // max(per_head_ms, 1e-6)))
    return max(1, min(int(largest), int(flat_heads) // 4, want))


class HostAttentionPipeline:
    """Attention on inputs and outputs that live in pinned host memory.

    Heads are independent, so the flat (batch x heads) axis is cut into chunks (see
    :func:`plan_chunks`) and five CUDA streams overlap: the upload of chunk i+1, its quantisation
    prepass (on a high-priority stream, so that its short kernels get SMs as soon as blocks of the
    running fused kernel retire), the fused kernel of chunk i and the download of chunk i-1.  The
    fused kernels alternate between two streams: a chunk's CTAs fill whole waves of SMs only by
    chance, and the next chunk's kernel then starts on the SMs its last, partial wave leaves idle.
    Device staging buffers (``slots`` per tensor) and the prepared calls (one per slot and chunk
    size, each with its workspace and output) are allocated once and re-used.

    ``op`` is the public function whose semantics are wanted, ``piper_attention`` or
    ``sage_attention_2pp``; keyword arguments are the ones that function takes.
    """

    def __init__(self, device, *, heads_per_chunk: int = 1, slots: int = 4, prepass_priority: int = -1):
        self.device = torch.device(device)
        self.heads_per_chunk = int(heads_per_chunk)
        self.n_slots = max(2, int(slots))  # staging slots: uploads run this many chunks ahead of the fused kernels
        self.up = torch.cuda.Stream(self.device)
        self.down = torch.cuda.Stream(self.device)
        self.prep = torch.cuda.Stream(self.device, priority=int(prepass_priority))
        self.run_b = torch.cuda.Stream(self.device)
        self._slots = None
        self._key = None
        self._calls = {}

    def _staging(self, q, k, v):
        key = (tuple(q.shape[2:]), tuple(k.shape[2:]), q.dtype)
        if self._key != key:
            n = self.heads_per_chunk
            mk = lambda t: torch.empty((n, *t.shape[2:]), dtype=t.dtype, device=self.device)  # noqa: E731
            self._slots = [{"q": mk(q), "k": mk(k), "v": mk(v), "free": None} for _ in range(self.n_slots)]
            self._key = key
            self._calls = {}
        return self._slots

    def _call(self, op, slot_index: int, n: int, kwargs: dict):
        """Prepared call on the first ``n`` heads of a staging slot, with ``op``'s own defaults."""
        from .attention._validation import validate_inputs
        from .attention.piper import default_center_value, should_sort_value_rows
        from .runtime import AttentionCall

        name = getattr(op, "__name__", str(op))
        if name not in ("piper_attention", "sage_attention_2pp"):
            raise ValueError(f"HostAttentionPipeline runs piper_attention or sage_attention_2pp, not {name}")
        key = (slot_index, n, name, tuple(sorted(kwargs.items())))
        call = self._calls.get(key)
        if call is None:
            slot = self._slots[slot_index]
            q, k, v = (slot[t][:n].unsqueeze(0) for t in ("q", "k", "v"))
            causal = bool(kwargs.get("is_causal", False))
            if name == "piper_attention":
                scale = validate_inputs("Piper Attention", q, k, v, kwargs.get("scale"), causal)
                center = kwargs.get("center_value")
                center = default_center_value(q, k, causal) if center is None else bool(center)
                sort = should_sort_value_rows(center_value=center, is_causal=causal, head_dim=q.shape[-1], key_length=k.shape[2])
                call = AttentionCall("piper", q, k, v, scale, causal, center=center, sort=sort)
            else:
                scale = validate_inputs("SageAttention2++", q, k, v, kwargs.get("scale"), causal)
                call = AttentionCall("sage2pp", q, k, v, scale, causal)
            call.drained = None
            self._calls[key] = call
        return call

    def __call__(self, op, q_host, k_host, v_host, out_host, *, copy_only: bool = False, **kwargs) -> torch.Tensor:
        """``copy_only=True`` performs the same uploads and downloads in the same order and with the
        same stream dependencies but launches no kernel: the time the host link alone needs (a
        measurement aid; ``out_host`` then receives whatever the staging outputs hold)."""
        b, h = q_host.shape[:2]
        flat = b * h
        fq, fk, fv = (t.flatten(0, 1) for t in (q_host, k_host, v_host))
        fo = out_host.view(flat, *out_host.shape[2:])
        slots = self._staging(q_host, k_host, v_host)
        main = torch.cuda.current_stream(self.device)
        for s in (self.up, self.down, self.prep, self.run_b):
            s.wait_stream(main)
        start = 0
        for i, n in enumerate(plan_chunks(flat, self.heads_per_chunk)):
            sl = slice(start, start + n)
            start += n
            slot = slots[i % self.n_slots]
            call = self._call(op, i % self.n_slots, n, kwargs)
            # Nothing hides the first chunk's upload: its K and V go first and their half of the
            # prepass (means, key order, codes) runs while its Q is still on the way.
            split_first = i == 0 and not copy_only
            with torch.cuda.stream(self.up):
                if slot["free"] is not None:
                    self.up.wait_event(slot["free"])  # the fused kernel that read this slot has finished
                slot["k"][:n].copy_(fk[sl], non_blocking=True)
                slot["v"][:n].copy_(fv[sl], non_blocking=True)
                kv_uploaded = torch.cuda.Event()
                if split_first:
                    kv_uploaded.record(self.up)
                slot["q"][:n].copy_(fq[sl], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(self.up)
            with torch.cuda.stream(self.prep):
                if split_first:
                    self.prep.wait_event(kv_uploaded)
                    call.prepare_kv()
                    self.prep.wait_event(uploaded)
                    call.requantize_q()
                else:
                    self.prep.wait_event(uploaded)
                    if not copy_only:
                        call.prepare()
                prepared = torch.cuda.Event()
                prepared.record(self.prep)
            run = main if i % 2 == 0 else self.run_b
            with torch.cuda.stream(run):
                run.wait_event(prepared)
                if call.drained is not None:
                    run.wait_event(call.drained)  # the download of this call's previous result has finished
                if not copy_only:
                    call.run()
                slot["free"] = torch.cuda.Event()
                slot["free"].record(run)
            with torch.cuda.stream(self.down):
                self.down.wait_event(slot["free"])
                fo[sl].copy_(call.out[0], non_blocking=True)
                call.drained = torch.cuda.Event()
                call.drained.record(self.down)
        for s in (self.down, self.up, self.prep, self.run_b):
            main.wait_stream(s)
        return out_host


def attention_from_host(op, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                        out_host: torch.Tensor, device, *, heads_per_chunk: int = 1, slots: int = 4, **kwargs) -> torch.Tensor:
    """One-shot form of :class:`HostAttentionPipeline` (allocates the staging buffers per call)."""
    return HostAttentionPipeline(device, heads_per_chunk=heads_per_chunk, slots=slots)(op, q_host, k_host, v_host, out_host, **kwargs)
