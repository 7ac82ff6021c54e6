"""Seeded synthetic inputs for the five benchmark configurations.

The reference benchmarks draw inputs with a seeded ``torch.randn``
(benchmarks/lib/attention.py:74-96 of the reference project); no dataset is involved.
Each configuration below reproduces the shapes, dtypes and value distributions named for
it.  Tensors are generated one (batch, head) at a time from ``seed * 1000 + flat_head`` so
that any sharding of heads across GPUs sees identical values.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    op: str  # "piper" | "sage2pp"
    batch: int
    heads: int
    q_len: int
    kv_len: int
    head_dim: int
    dtype: torch.dtype
    causal: bool
    center: bool | None  # None: the public default policy decides
    seed: int
    note: str

    @property
    def flat_heads(self) -> int:
        return self.batch * self.heads

    def ops(self, flat_heads: int | None = None) -> float:
        """4*B*H*Sq*Sk*D, the metric's operation count (causal uses the same full formula)."""
        n = self.flat_heads if flat_heads is None else flat_heads
        return 4.0 * n * self.q_len * self.kv_len * self.head_dim


WORKLOADS = {
    "c1": Workload("c1", "piper", 1, 8, 1024, 1024, 64, torch.float16, False, False, 1,
                   "piper non-causal D64 S1024 fp16, K channel bias N(0,0.5)"),
    "c2": Workload("c2", "piper", 2, 24, 4096, 4096, 128, torch.bfloat16, False, None, 2,
                   "piper non-causal D128 S4096 bf16, V bias N(0,2) per (head,feature): default centering"),
    "c3": Workload("c3", "piper", 4, 32, 8192, 8192, 128, torch.float16, True, False, 3,
                   "piper causal D128 S8192 fp16, K channel bias N(0,1); prefill shape"),
    "c4": Workload("c4", "piper", 1, 40, 32760, 32760, 128, torch.bfloat16, False, None, 4,
                   "piper non-causal centered long-key D128 S32760 bf16 (video-DiT token count), sorted key order"),
    "c5": Workload("c5", "sage2pp", 2, 16, 4096, 16384, 64, torch.float16, False, None, 5,
                   "sage2pp rectangular non-causal D64 Sq4096 Sk16384 fp16, K/V interleaved (stride 2*D)"),
}


def _head(w: Workload, flat_head: int, device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(w.seed * 1000 + flat_head)
    shared = torch.Generator(device=device).manual_seed(w.seed * 1000 + 999)  # values shared by all heads
    d = w.head_dim
    rn = lambda *s, gen=g: torch.randn(*s, generator=gen, device=device, dtype=torch.float32)  # noqa: E731
    q = rn(w.q_len, d)
    k = rn(w.kv_len, d)
    v = rn(w.kv_len, d)
    if w.name == "c1":
        k = k + 0.5 * rn(1, d, gen=shared)
    elif w.name == "c2":
        v = v + 2.0 * rn(1, d)
    elif w.name == "c3":
        k = k + rn(1, d, gen=shared)
    elif w.name == "c4":
        spread = 0.5 + 1.5 * torch.rand(1, d, generator=shared, device=device)
        v = v * spread + 3.0 * rn(1, d, gen=shared)
    elif w.name == "c5":
        k = k + rn(1, d, gen=shared)
    return q.to(w.dtype), k.to(w.dtype), v.to(w.dtype)


def make_inputs(w: Workload, device, heads: range | None = None):
    """q, k, v for the flat heads in ``heads`` (default: all), shaped [1, n, S, D] when a
    subset is asked for, else [B, H, S, D].  For c5, k and v are the two halves of one
    interleaved buffer (sequence stride 2*D), as in the configuration's description."""
    sel = range(w.flat_heads) if heads is None else heads
    n = len(sel)
    q = torch.empty(n, w.q_len, w.head_dim, dtype=w.dtype, device=device)
    if w.name == "c5":
        kv = torch.empty(n, w.kv_len, 2, w.head_dim, dtype=w.dtype, device=device)
        k, v = kv[:, :, 0, :], kv[:, :, 1, :]
    else:
        k = torch.empty(n, w.kv_len, w.head_dim, dtype=w.dtype, device=device)
        v = torch.empty_like(k)
    for i, fh in enumerate(sel):
        qi, ki, vi = _head(w, fh, device)
        q[i], k[i], v[i] = qi, ki, vi
    if heads is None:
        shape = lambda t: t.unflatten(0, (w.batch, w.heads))  # noqa: E731
    else:
        shape = lambda t: t.unsqueeze(0)  # noqa: E731
    return shape(q), shape(k), shape(v)
