"""Oracle for the Q4_K x Q8_K quantized projection (test infrastructure).

Reference sources followed: examples/kernels/quantization/quantized_projection.py:5-19 (the
program) and doc/dsl/quantized-operations.en.md sections 2-4 (record formats, dot numerics,
Q8_K quantization numerics), restated with numpy float32 arithmetic (one rounding per
operation, no fused multiply-add).

PARITY UNPINNED: the reference holds no golden vectors and no executable CPU implementation
of these operations in its tree (its comparison runs a RISC-V build on a remote host), so this
restatement of the published record arithmetic is the only checker.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def q8_k_quantize(values: np.ndarray) -> np.ndarray:
    """f32 [G, 256] -> u8 [G, 292]: ds f32 | q i8[256] | bsum i16[16] (section 4)."""
    values = np.asarray(values, dtype=F32)
    records = np.zeros((values.shape[0], 292), dtype=np.uint8)
    for g, block in enumerate(values):
        high, low = block.max(), block.min()
        extreme = low if abs(low) >= abs(high) else high          # the minimum wins ties
        if extreme == 0:
            continue                                               # ds = +0, q = 0, bsum = 0
        inverse = F32(-127.0) / F32(extreme)
        ds = F32(1.0) / inverse
        scaled = (block * inverse).astype(F32)
        q = np.clip(np.rint(scaled), -128, 127).astype(np.int8)    # rint: nearest even
        records[g, 0:4] = np.frombuffer(F32(ds).tobytes(), dtype=np.uint8)
        records[g, 4:260] = q.view(np.uint8)
        records[g, 260:292] = q.astype(np.int16).reshape(16, 16).sum(axis=1).astype('<i2').view(np.uint8)
    return records


def q4_k_fields(record: np.ndarray):
    """u8 [144] -> (d, dmin as f32, sc[8], m[8], q[256]) (section 2)."""
    a = record.astype(np.int64)
    d = F32(np.frombuffer(record[0:2].tobytes(), dtype='<f2')[0])
    dmin = F32(np.frombuffer(record[2:4].tobytes(), dtype='<f2')[0])
    fields = []
    for r in (0, 1):
        low = [a[4 + 4 * r + i] & 63 for i in range(4)]
        high = [((a[12 + t] >> (4 * r)) & 15) | ((a[4 + 4 * r + t] >> 6) << 4) for t in range(4)]
        fields.append(np.array(low + high, dtype=np.int64))
    i = np.arange(256)
    packed = a[16 + 32 * (i // 64) + (i % 32)]
    q = (packed >> np.where(i % 64 < 32, 0, 4)) & 15
    return d, dmin, fields[0], fields[1], q


def quantized_dot(weights: np.ndarray, activation_records: np.ndarray) -> np.float32:
    """u8 [G, 144] . u8 [G, 292] -> f32 (section 3); records are added in increasing order."""
    result = F32(0.0)
    for w, x in zip(weights, activation_records):
        d, dmin, sc, m, wq = q4_k_fields(w)
        ds = np.frombuffer(x[0:4].tobytes(), dtype='<f4')[0]
        xq = x[4:260].view(np.int8).astype(np.int64)
        bsum = np.frombuffer(x[260:292].tobytes(), dtype='<i2').astype(np.int64)
        s_total = int(sum(sc[s] * int((wq[32 * s:32 * s + 32] * xq[32 * s:32 * s + 32]).sum()) for s in range(8)))
        t_total = int(sum(m[s] * (bsum[2 * s] + bsum[2 * s + 1]) for s in range(8)))
        p = F32(d * F32(s_total))
        n = F32(dmin * F32(t_total))
        result = F32(result + F32(F32(ds) * F32(p - n)))
    return result


def quantized_projection(weights: np.ndarray, activation: np.ndarray) -> np.ndarray:
    """weights u8 [N, G, 144], activation f32 [G, 256] -> f32 [N]."""
    records = q8_k_quantize(activation)
    return np.array([quantized_dot(row, records) for row in weights], dtype=F32)
