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


# ------------------------------------------------------------------ seeded model weights
def encoder_weight_shapes(layers: int = 24, d_model: int = 1024, heads: int = 8, ff: int = 4096, conv_kernel: int = 9,
                          sub_channels: int = 256, mels: int = 128) -> dict:
    """Names and shapes of the FastConformer encoder tensors (the names sb_model_load expects)."""
    C, d, k = sub_channels, d_model, conv_kernel
    f_out = mels // 8
    s = {
        "subsampling.layers.0.weight": (C, 1, 3, 3), "subsampling.layers.0.bias": (C,),
        "subsampling.layers.2.weight": (C, 1, 3, 3), "subsampling.layers.2.bias": (C,),
        "subsampling.layers.3.weight": (C, C, 1, 1), "subsampling.layers.3.bias": (C,),
        "subsampling.layers.5.weight": (C, 1, 3, 3), "subsampling.layers.5.bias": (C,),
        "subsampling.layers.6.weight": (C, C, 1, 1), "subsampling.layers.6.bias": (C,),
        "subsampling.linear.weight": (d, C * f_out), "subsampling.linear.bias": (d,),
    }
    for i in range(layers):
        p = f"layers.{i}."
        for ffn in ("feed_forward1", "feed_forward2"):
            s[p + ffn + ".linear1.weight"] = (ff, d)
            s[p + ffn + ".linear1.bias"] = (ff,)
            s[p + ffn + ".linear2.weight"] = (d, ff)
            s[p + ffn + ".linear2.bias"] = (d,)
        for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
            s[p + "self_attn." + proj + ".weight"] = (d, d)
            s[p + "self_attn." + proj + ".bias"] = (d,)
        s[p + "self_attn.relative_k_proj.weight"] = (d, d)
        s[p + "self_attn.bias_u"] = (heads, d // heads)
        s[p + "self_attn.bias_v"] = (heads, d // heads)
        s[p + "conv.pointwise_conv1.weight"] = (2 * d, d, 1)
        s[p + "conv.pointwise_conv1.bias"] = (2 * d,)
        s[p + "conv.depthwise_conv.weight"] = (d, 1, k)
        s[p + "conv.depthwise_conv.bias"] = (d,)
        for n in ("weight", "bias", "running_mean", "running_var"):
            s[p + "conv.norm." + n] = (d,)
        s[p + "conv.pointwise_conv2.weight"] = (d, d, 1)
        s[p + "conv.pointwise_conv2.bias"] = (d,)
        for ln in ("norm_feed_forward1", "norm_self_att", "norm_conv", "norm_feed_forward2", "norm_out"):
            s[p + ln + ".weight"] = (d,)
            s[p + ln + ".bias"] = (d,)
    return s


def seeded_encoder_weights(layers: int, seed: int, std: float = 0.02, plain_norms: bool = True, **shape_kw) -> dict:
    """N(0, std) for every matrix, bias and u/v.  plain_norms=True: LayerNorm gamma 1 / beta 0 and
    BatchNorm gamma 1, beta 0, mean 0, var 1 (the benchmark configuration); False: seeded
    non-trivial values so that tests exercise every parameter."""
    w = {}
    for name, shape in encoder_weight_shapes(layers, **shape_kw).items():
        is_norm = ".norm" in name or "norm_" in name
        if is_norm:
            if plain_norms:
                v = np.ones(shape, np.float32) if name.endswith(("weight", "running_var")) else np.zeros(shape, np.float32)
            elif name.endswith("running_var"):
                v = 0.5 + np.abs(normal_tensor(name, shape, 0.5, seed))
            elif name.endswith("weight"):
                v = 1.0 + normal_tensor(name, shape, 0.1, seed)
            else:
                v = normal_tensor(name, shape, 0.1, seed)
        else:
            v = normal_tensor(name, shape, std, seed)
        w[name] = v.astype(np.float32)
    return w


DECODER_SHAPES = {
    "predictor.embedding": (1025, 640),
    "predictor.lstm.weight_ih": (2, 2560, 640),
    "predictor.lstm.weight_hh": (2, 2560, 640),
    "predictor.lstm.bias_ih": (2, 2560),
    "predictor.lstm.bias_hh": (2, 2560),
    "joint.enc.weight": (640, 1024),
    "joint.enc.bias": (640,),
    "joint.pred.weight": (640, 640),
    "joint.pred.bias": (640,),
    "joint.out.weight": (1030, 640),
    "joint.out.bias": (1030,),
}


def seeded_decoder_weights(seed: int, std: float = 0.05) -> dict:
    """Predictor / joint weights: N(0, std) per tensor, named as sb_model_load expects."""
    return {k: normal_tensor(k, shp, std, seed) for k, shp in DECODER_SHAPES.items()}


def seeded_model(layers: int, encoder_seed: int = 2, decoder_seed: int = 3) -> dict:
    """The benchmark model: encoder N(0, 0.02) with identity norms, predictor / joint N(0, 0.05)."""
    w = seeded_encoder_weights(layers, seed=encoder_seed, std=0.02, plain_norms=True)
    w.update(seeded_decoder_weights(decoder_seed, std=0.05))
    return w


# ---------------------------------------------------------------------------- voice-activity network
VAD_SHAPES = {
    "stft.forward_basis_buffer": (258, 1, 256),
    "encoder.0.reparam_conv.weight": (128, 129, 3), "encoder.0.reparam_conv.bias": (128,),
    "encoder.1.reparam_conv.weight": (64, 128, 3), "encoder.1.reparam_conv.bias": (64,),
    "encoder.2.reparam_conv.weight": (64, 64, 3), "encoder.2.reparam_conv.bias": (64,),
    "encoder.3.reparam_conv.weight": (128, 64, 3), "encoder.3.reparam_conv.bias": (128,),
    "decoder.rnn.weight_ih": (512, 128), "decoder.rnn.weight_hh": (512, 128),
    "decoder.rnn.bias_ih": (512,), "decoder.rnn.bias_hh": (512,),
    "decoder.decoder.2.weight": (1, 128, 1), "decoder.decoder.2.bias": (1,),
}


def vad_stft_basis() -> np.ndarray:
    """Hann-windowed DFT rows of length 256: 129 real (cos) rows, then 129 imaginary (-sin) rows."""
    n = np.arange(256, dtype=np.float64)
    window = 0.5 - 0.5 * np.cos(2.0 * np.pi * n / 256.0)
    k = np.arange(129, dtype=np.float64)[:, None]
    ang = 2.0 * np.pi * k * n[None, :] / 256.0
    return np.concatenate([np.cos(ang) * window, -np.sin(ang) * window]).astype(np.float32).reshape(258, 1, 256)


def seeded_vad_weights(seed: int) -> dict:
    """Random weights with the shapes of the voice-activity network (the reference's network file is not
    distributed with it): convolutions N(0, 1.4 / sqrt(fan_in)), recurrent matrices N(0, 0.12), output layer
    N(0, 0.5); the Fourier basis is the true Hann-windowed DFT."""
    w = {}
    for name, shape in VAD_SHAPES.items():
        if name == "stft.forward_basis_buffer":
            w[name] = vad_stft_basis()
        elif name.startswith("encoder.") and name.endswith("weight"):
            w[name] = normal_tensor("vad." + name, shape, 1.4 / np.sqrt(shape[1] * shape[2]), seed)
        elif name.startswith("decoder.rnn.weight"):
            w[name] = normal_tensor("vad." + name, shape, 0.12, seed)
        elif name == "decoder.decoder.2.weight":
            w[name] = normal_tensor("vad." + name, shape, 0.5, seed)
        else:
            w[name] = normal_tensor("vad." + name, shape, 0.1, seed)
    return w


def energy_vad_weights(gain: float = 20.0, offset: float = 2.0) -> dict:
    """Weights that turn the network into an energy detector, so that end-to-end runs of the VAD mode see
    probabilities near 1 on sound and near 0 on silence: channel 0 of every layer carries the mean spectral
    magnitude E of the window, the LSTM cell has input and output gates open and the forget gate shut, the cell
    candidate is tanh(gain * E - offset), and the output layer is sigmoid(20 * relu(h_0) - 4)."""
    w = {name: np.zeros(shape, np.float32) for name, shape in VAD_SHAPES.items()}
    w["stft.forward_basis_buffer"] = vad_stft_basis()
    w["encoder.0.reparam_conv.weight"][0, :, 1] = 1.0 / 129.0
    w["encoder.1.reparam_conv.weight"][0, 0, :] = 1.0 / 3.0
    w["encoder.2.reparam_conv.weight"][0, 0, 1:] = 0.5
    w["encoder.3.reparam_conv.weight"][0, 0, 1] = 1.0
    b = w["decoder.rnn.bias_ih"]
    b[0:128] = 10.0      # input gate open
    b[128:256] = -10.0   # forget gate shut
    b[256:384] = -offset
    b[384:512] = 10.0    # output gate open
    w["decoder.rnn.weight_ih"][256:384, 0] = gain
    w["decoder.decoder.2.weight"][0, 0, 0] = 20.0
    w["decoder.decoder.2.bias"][0] = -4.0
    return w


def sparse_speech_audio(n_samples: int, seed: int, speech_seconds=(2.0, 20.0), silence_seconds=(1.0, 6.0)) -> np.ndarray:
    """A recording for the VAD mode: stretches of `long_audio`-like sound (durations U(speech_seconds)) separated by
    near-silence (N(0, 1e-4) noise, durations U(silence_seconds))."""
    rng = np.random.default_rng(seed)
    out = rng.normal(0.0, 1e-4, n_samples).astype(np.float32)
    pos = int(rng.uniform(*silence_seconds) * SAMPLE_RATE)
    k = 0
    while pos < n_samples:
        n = min(int(rng.uniform(*speech_seconds) * SAMPLE_RATE), n_samples - pos)
        out[pos:pos + n] += clip_audio(n, seed * 1000 + k)
        pos += n + int(rng.uniform(*silence_seconds) * SAMPLE_RATE)
        k += 1
    return out
