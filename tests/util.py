"""Shared helpers for the parity tests."""
import numpy as np


def rel_err(got: np.ndarray, ref: np.ndarray):
    """(max|got-ref| / max|ref|, rms(got-ref) / rms(ref)) — the error measure used for every
    matmul tolerance in this suite.  Element-wise relative error is meaningless here because
    outputs cross zero."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = max(np.abs(ref).max(), 1e-30)
    rms = max(np.sqrt((ref ** 2).mean()), 1e-30)
    d = got - ref
    return float(np.abs(d).max() / den), float(np.sqrt((d ** 2).mean()) / rms)


def describe_mismatch(got: np.ndarray, ref: np.ndarray, limit: int = 8) -> str:
    got = np.asarray(got)
    ref = np.asarray(ref)
    bad = np.argwhere(~np.isclose(got, ref, rtol=1e-4, atol=1e-6 * max(np.abs(ref).max(), 1e-30)))
    lines = [f"{len(bad)} of {got.size} elements differ; first {min(limit, len(bad))}:"]
    for idx in bad[:limit]:
        t = tuple(int(i) for i in idx)
        lines.append(f"  {t}: got {got[t]!r} want {ref[t]!r}")
    return "\n".join(lines)


def seed_of(*parts) -> int:
    """Deterministic small integer from test parameters (Python's str hash is salted per process)."""
    import zlib

    return zlib.crc32(repr(parts).encode()) % 1000
