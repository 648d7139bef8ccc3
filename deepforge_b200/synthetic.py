"""Seeded synthetic inputs shared by the tests and the benchmark.

Every element is a pure function of (seed, stream, index):
    r = splitmix64(seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + index)
    u = (r >> 11) * 2^-53
uniform[a, b) = a + (b - a) * u; normal via Box-Muller on indices 2i, 2i+1.
`stream` is normally the tensor's UID. Values are produced in f64, cast to f32,
and rounded to bf16 (nearest even) by the caller where the tensor is bf16.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint64, copy=True)
    with np.errstate(over="ignore"):
        x += np.uint64(0x9E3779B97F4A7C15)
        z = x
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def raw_u64(seed: int, stream: int, count: int, start: int = 0) -> np.ndarray:
    base = (seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF
    with np.errstate(over="ignore"):
        index = np.arange(start, start + count, dtype=np.uint64) + np.uint64(base)
    return splitmix64(index)


def unit(seed: int, stream: int, count: int, start: int = 0) -> np.ndarray:
    return (raw_u64(seed, stream, count, start) >> np.uint64(11)).astype(np.float64) * (2.0 ** -53)


def uniform(seed: int, stream: int, count: int, low: float, high: float) -> np.ndarray:
    return (low + (high - low) * unit(seed, stream, count)).astype(np.float32)


def normal(seed: int, stream: int, count: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    pairs = (count + 1) // 2
    u = unit(seed, stream, 2 * pairs)
    u1 = np.maximum(u[0::2], 2.0 ** -53)
    u2 = u[1::2]
    radius = np.sqrt(-2.0 * np.log(u1))
    out = np.empty(2 * pairs, dtype=np.float64)
    out[0::2] = radius * np.cos(2.0 * np.pi * u2)
    out[1::2] = radius * np.sin(2.0 * np.pi * u2)
    return (mean + std * out[:count]).astype(np.float32)


def normal_on_device(device, seed: int, stream: int, count: int, bf16: bool = True, chunk: int = 1 << 24):
    """The N(0, 1) stream of normal() / the workloads' generators evaluated with torch on `device`, for tensors too
    large to draw on the host in reasonable time (the paged KV pools): the same splitmix64 words (two's-complement
    int64 arithmetic wraps like uint64), the same Box-Muller pairs in f64, cast to f32 and rounded to bf16. The
    device's f64 log / cos / sin may differ from the host's in the last place, which survives the rounding to bf16
    with probability ~2^-40 per element. `count` must be even. Returns a torch tensor (bf16 or f32)."""
    import torch
    assert count % 2 == 0
    base = (seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF

    def signed(value: int) -> int:
        value &= 0xFFFFFFFFFFFFFFFF
        return value - (1 << 64) if value >= (1 << 63) else value

    def shift_right(z, bits: int):
        return (z >> bits) & ((1 << (64 - bits)) - 1)  # logical shift of the uint64 the int64 stands for

    out = torch.empty(count, dtype=torch.bfloat16 if bf16 else torch.float32, device=device)
    for start in range(0, count, chunk):
        n = min(chunk, count - start)
        z = torch.arange(n, dtype=torch.int64, device=device) + signed(base + start + 0x9E3779B97F4A7C15)
        z = (z ^ shift_right(z, 30)) * signed(0xBF58476D1CE4E5B9)
        z = (z ^ shift_right(z, 27)) * signed(0x94D049BB133111EB)
        z = z ^ shift_right(z, 31)
        u = shift_right(z, 11).to(torch.float64) * (2.0 ** -53)
        u1 = torch.clamp(u[0::2], min=2.0 ** -53)
        radius = torch.sqrt(-2.0 * torch.log(u1))
        angle = 2.0 * np.pi * u[1::2]
        values = torch.stack((radius * torch.cos(angle), radius * torch.sin(angle)), dim=1).reshape(-1)
        out[start:start + n] = values.to(torch.float32).to(out.dtype)
    return out


def integers(seed: int, stream: int, count: int, low: int, high_inclusive: int) -> np.ndarray:
    span = np.uint64(high_inclusive - low + 1)
    return (raw_u64(seed, stream, count) % span).astype(np.int64) + low


def outlier_mask(seed: int, stream: int, count: int, one_in: int = 100) -> np.ndarray:
    return (raw_u64(seed, stream + 0x5151, count) % np.uint64(one_in)) == 0


def permutation_prefix(seed: int, stream: int, population: int, take: int) -> np.ndarray:
    """First `take` entries of a seeded Fisher-Yates shuffle of range(population)."""
    values = np.arange(population, dtype=np.int64)
    draws = raw_u64(seed, stream, take)
    for i in range(take):
        j = i + int(draws[i] % np.uint64(population - i))
        values[i], values[j] = values[j], values[i]
    return values[:take].copy()


def to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns, round to nearest even (NaN kept quiet)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = ((bits.astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    rounded[nan] = ((bits[nan] >> 16) | 0x0040).astype(np.uint16)
    return rounded


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(values: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(to_bf16_bits(values)).reshape(values.shape)
