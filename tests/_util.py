"""Helpers shared by the tests: golden fixture loading and 16-bit <-> float32 conversion."""

from __future__ import annotations

from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"


def widen16(bits: np.ndarray, dtype: str) -> np.ndarray:
    """uint16 bit patterns of float16 / bfloat16 values -> float32."""
    bits = np.asarray(bits, dtype=np.uint16)
    if dtype == "float16":
        return bits.view(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        return (bits.astype(np.uint32) << 16).view(np.float32)
    raise ValueError(dtype)


def short(dtype: str) -> str:
    return {"float16": "f16", "bfloat16": "bf16"}[dtype]


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz", allow_pickle=False) as z:
        rec = {k: z[k] for k in z.files}
    for key in ("kind", "dtype"):
        rec[key] = str(rec[key])
    for key in ("causal", "center", "sort"):
        if key in rec:
            rec[key] = bool(rec[key])
    rec["scale"] = float(rec["scale"])
    for t in "qkv":
        rec[t + "f"] = widen16(rec[t], rec["dtype"])
    return rec


def golden_names(kind: str) -> list[str]:
    return sorted(p.stem for p in GOLDEN.glob(f"{kind}_*.npz"))


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))
