"""Seeded synthetic inputs and weights with the shapes of the benchmark configurations.

The reference measures on audio and model files that are not distributed with
it; these generators stand in for them.  Audio is mono 16 kHz f32: a sum of
five sinusoids (frequencies U(100, 4000) Hz, phases U(0, 2*pi), amplitude 0.1
each) plus N(0, sigma = 0.01) noise, clipped to [-1, 1].  Weights are N(0, std)
per tensor from a per-tensor seed.
"""
from __future__ import annotations

import zlib

import numpy as np

SAMPLE_RATE = 16000


def clip_audio(n_samples: int, seed: int, silent: bool = False) -> np.ndarray:
    """One clip (numpy; used for parity-sized inputs)."""
    if silent:
        return np.zeros(n_samples, np.float32)
    rng = np.random.default_rng(seed)
    freqs = rng.uniform(100.0, 4000.0, 5)
    phases = rng.uniform(0.0, 2.0 * np.pi, 5)
    t = np.arange(n_samples, dtype=np.float64) / SAMPLE_RATE
    x = np.zeros(n_samples, np.float64)
    for f, p in zip(freqs, phases):
        x += 0.1 * np.sin(2.0 * np.pi * f * t + p)
    x += rng.normal(0.0, 0.01, n_samples)
    return np.clip(x, -1.0, 1.0).astype(np.float32)


def clip_batch(n_clips: int, n_samples: int, base_seed: int = 0, silent_every: int = 10,
               silent_phase: int = 3) -> np.ndarray:
    """[n_clips, n_samples]; clips with index % silent_every == silent_phase are all-zero."""
    out = np.empty((n_clips, n_samples), np.float32)
    for c in range(n_clips):
        silent = silent_every > 0 and c % silent_every == silent_phase
        out[c] = clip_audio(n_samples, base_seed + c, silent)
    return out


def clip_batch_torch(n_clips: int, n_samples: int, base_seed: int, device, silent_every: int = 10,
                     silent_phase: int = 3):
    """Same distribution generated with torch on `device` (bulk benchmark inputs).
    The sample values differ from `clip_batch` (different generator)."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(base_seed)
    freqs = torch.empty(n_clips, 5, device=device).uniform_(100.0, 4000.0, generator=g)
    phases = torch.empty(n_clips, 5, device=device).uniform_(0.0, 2.0 * np.pi, generator=g)
    out = torch.empty(n_clips, n_samples, device=device, dtype=torch.float32)
    t = torch.arange(n_samples, device=device, dtype=torch.float32) / SAMPLE_RATE
    step = max(1, (64 << 20) // max(n_samples, 1))
    for c0 in range(0, n_clips, step):
        c1 = min(n_clips, c0 + step)
        x = torch.zeros(c1 - c0, n_samples, device=device)
        for j in range(5):
            x += 0.1 * torch.sin(2.0 * np.pi * freqs[c0:c1, j:j + 1] * t[None, :] + phases[c0:c1, j:j + 1])
        x += 0.01 * torch.randn(c1 - c0, n_samples, device=device, generator=g)
        out[c0:c1] = x.clamp_(-1.0, 1.0)
    if silent_every > 0:
        idx = torch.arange(n_clips, device=device)
        out[idx % silent_every == silent_phase] = 0.0
    return out


def long_audio(n_samples: int, seed: int) -> np.ndarray:
    """'Speech' segments of U(1, 20) s (fresh sinusoids each) alternating with
    U(0.5, 5) s of zeros, until n_samples (numpy; parity-sized)."""
    rng = np.random.default_rng(seed)
    out = np.zeros(n_samples, np.float32)
    pos = 0
    k = 0
    while pos < n_samples:
        seg = int(rng.uniform(1.0, 20.0) * SAMPLE_RATE)
        end = min(n_samples, pos + seg)
        out[pos:end] = clip_audio(end - pos, int(rng.integers(1 << 31)) + k)
        pos = end + int(rng.uniform(0.5, 5.0) * SAMPLE_RATE)
        k += 1
    return out


def long_audio_torch(n_samples: int, seed: int, device):
    """Bulk version of `long_audio` on `device` (different generator, same distribution)."""
    import torch

    rng = np.random.default_rng(seed)
    bounds = []
    pos = 0
    while pos < n_samples:
        seg = int(rng.uniform(1.0, 20.0) * SAMPLE_RATE)
        end = min(n_samples, pos + seg)
        bounds.append((pos, end))
        pos = end + int(rng.uniform(0.5, 5.0) * SAMPLE_RATE)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = torch.zeros(n_samples, device=device, dtype=torch.float32)
    for (a, b) in bounds:
        n = b - a
        freqs = torch.empty(5, device=device).uniform_(100.0, 4000.0, generator=g)
        phases = torch.empty(5, device=device).uniform_(0.0, 2.0 * np.pi, generator=g)
        t = torch.arange(n, device=device, dtype=torch.float32) / SAMPLE_RATE
        x = 0.01 * torch.randn(n, device=device, generator=g)
        for j in range(5):
            x += 0.1 * torch.sin(2.0 * np.pi * freqs[j] * t + phases[j])
        out[a:b] = x.clamp_(-1.0, 1.0)
    return out


def normal_tensor(name: str, shape, std: float, seed: int) -> np.ndarray:
    """N(0, std) f32 tensor from a seed derived from (seed, name); stable across runs."""
    s = (zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0xFFFFFFFF
    rng = np.random.default_rng(s)
    return (rng.standard_normal(int(np.prod(shape)), dtype=np.float32) * np.float32(std)).reshape(shape)
