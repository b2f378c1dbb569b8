"""fp32 CPU oracle of the FastConformer encoder.  TEST INFRASTRUCTURE ONLY.

The reference runs its encoder as an opaque CoreML blob (src/models.rs:5,
I/O contract src/coreml.rs:75-135); its arithmetic is not in the reference
tree, so this oracle is a definition, not a restatement, and its parity with
the reference's blob is UNPINNED.  What it is pinned against is the published
FastConformer structure as implemented, independently, by the installed
`transformers` package (`ParakeetEncoder`): tests/test_oracle_encoder.py loads
the same seeded weights into both and compares outputs.

Structure (Parakeet-TDT-0.6B-v2 shape: 128 mels, 256 sub-sampling channels,
d_model 1024, 8 heads, FF 4096, depthwise k = 9, 24 blocks):
  sub-sampling  conv2d(1->C, k3, s2, p1) + ReLU, then twice [depthwise conv2d(k3, s2, p1),
                pointwise 1x1, ReLU]; flatten (channel-major: c * F + f) -> Linear -> d_model;
                optional input scale sqrt(d_model)
  positions     sinusoidal table for relative positions T'-1 .. -(T'-1), sin/cos interleaved
  block         x += 0.5 FF(LN x); x += MHA_rel(LN x); x += Conv(LN x); x += 0.5 FF(LN x); x = LN x
  MHA_rel       scores = ((q + u) k^T + rel_shift((q + v) (W_r pos)^T)) / sqrt(d_head), softmax, V
  Conv          pointwise (d -> 2d), GLU, depthwise k9 'same', BatchNorm (eval), SiLU, pointwise
Each clip is processed alone with its exact length (no padding), which equals
the masked, padded batch of the library implementation.

Weight names are those of `ParakeetEncoder.state_dict()`.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from scriptrs_b200 import synth


class EncoderConfig:
    def __init__(self, layers=24, d_model=1024, heads=8, ff=4096, conv_kernel=9, sub_channels=256, mels=128,
                 scale_input=False):
        self.layers, self.d_model, self.heads, self.ff = layers, d_model, heads, ff
        self.conv_kernel, self.sub_channels, self.mels, self.scale_input = conv_kernel, sub_channels, mels, scale_input


def subsampled_length(t: int) -> int:
    for _ in range(3):
        t = (t - 1) // 2 + 1
    return t


def _shape_kw(cfg: EncoderConfig):
    return dict(d_model=cfg.d_model, heads=cfg.heads, ff=cfg.ff, conv_kernel=cfg.conv_kernel,
                sub_channels=cfg.sub_channels, mels=cfg.mels)


def weight_shapes(cfg: EncoderConfig):
    return synth.encoder_weight_shapes(cfg.layers, **_shape_kw(cfg))


def seeded_weights(cfg: EncoderConfig, seed: int, std: float = 0.02, plain_norms: bool = True):
    """Seeded weights of scriptrs_b200.synth for this configuration (same tensors for oracle and library)."""
    return synth.seeded_encoder_weights(cfg.layers, seed, std, plain_norms, **_shape_kw(cfg))


def rel_positions(t: int, d_model: int) -> torch.Tensor:
    """[2t-1, d_model]: rows for relative positions t-1 .. -(t-1); sin/cos interleaved."""
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d_model, 2, dtype=torch.float32) / d_model))
    pos = torch.arange(t - 1, -t, -1, dtype=torch.float32)
    ang = pos[:, None] * inv_freq[None, :]
    return torch.stack([ang.sin(), ang.cos()], dim=-1).reshape(2 * t - 1, d_model)


def _t(w, name):
    return torch.from_numpy(np.ascontiguousarray(w[name]))


def subsampling(w, feats: torch.Tensor, cfg: EncoderConfig) -> torch.Tensor:
    x = feats[None, None]  # [1, 1, T, mels]
    x = F.relu(F.conv2d(x, _t(w, "subsampling.layers.0.weight"), _t(w, "subsampling.layers.0.bias"), stride=2, padding=1))
    for dw, pw in ((2, 3), (5, 6)):
        x = F.conv2d(x, _t(w, f"subsampling.layers.{dw}.weight"), _t(w, f"subsampling.layers.{dw}.bias"), stride=2,
                     padding=1, groups=cfg.sub_channels)
        x = F.relu(F.conv2d(x, _t(w, f"subsampling.layers.{pw}.weight"), _t(w, f"subsampling.layers.{pw}.bias")))
    x = x.transpose(1, 2).reshape(1, x.shape[2], -1)  # [1, T', C * F'] channel-major
    x = F.linear(x, _t(w, "subsampling.linear.weight"), _t(w, "subsampling.linear.bias"))
    if cfg.scale_input:
        x = x * math.sqrt(cfg.d_model)
    return x[0]


def _ln(w, p, x):
    return F.layer_norm(x, (x.shape[-1],), _t(w, p + ".weight"), _t(w, p + ".bias"), 1e-5)


def _ff(w, p, x):
    h = F.silu(F.linear(x, _t(w, p + ".linear1.weight"), _t(w, p + ".linear1.bias")))
    return F.linear(h, _t(w, p + ".linear2.weight"), _t(w, p + ".linear2.bias"))


def _attention(w, p, x, pos, cfg: EncoderConfig):
    t, d = x.shape
    h, dh = cfg.heads, d // cfg.heads
    q = F.linear(x, _t(w, p + ".q_proj.weight"), _t(w, p + ".q_proj.bias")).view(t, h, dh).transpose(0, 1)
    k = F.linear(x, _t(w, p + ".k_proj.weight"), _t(w, p + ".k_proj.bias")).view(t, h, dh).transpose(0, 1)
    v = F.linear(x, _t(w, p + ".v_proj.weight"), _t(w, p + ".v_proj.bias")).view(t, h, dh).transpose(0, 1)
    r = F.linear(pos, _t(w, p + ".relative_k_proj.weight")).view(2 * t - 1, h, dh).transpose(0, 1)  # [h, 2t-1, dh]
    qu = q + _t(w, p + ".bias_u")[:, None, :]
    qv = q + _t(w, p + ".bias_v")[:, None, :]
    ac = qu @ k.transpose(1, 2)                       # [h, t, t]
    bd_full = qv @ r.transpose(1, 2)                  # [h, t, 2t-1], column p <-> relative position t-1-p
    # rel_shift: score(i, j) uses relative position i - j, i.e. column t - 1 - (i - j)
    idx = (t - 1) - (torch.arange(t)[:, None] - torch.arange(t)[None, :])
    bd = torch.gather(bd_full, 2, idx[None].expand(h, t, t))
    att = torch.softmax((ac + bd) / math.sqrt(dh), dim=-1)
    o = (att @ v).transpose(0, 1).reshape(t, d)
    return F.linear(o, _t(w, p + ".o_proj.weight"), _t(w, p + ".o_proj.bias"))


def _conv_module(w, p, x, cfg: EncoderConfig):
    d = x.shape[1]
    y = F.linear(x, _t(w, p + ".pointwise_conv1.weight")[:, :, 0], _t(w, p + ".pointwise_conv1.bias"))
    y = y[:, :d] * torch.sigmoid(y[:, d:])            # GLU over channels
    y = F.conv1d(y.t()[None], _t(w, p + ".depthwise_conv.weight"), _t(w, p + ".depthwise_conv.bias"),
                 padding=(cfg.conv_kernel - 1) // 2, groups=d)[0].t()
    y = (y - _t(w, p + ".norm.running_mean")) / torch.sqrt(_t(w, p + ".norm.running_var") + 1e-5)
    y = y * _t(w, p + ".norm.weight") + _t(w, p + ".norm.bias")
    y = F.silu(y)
    return F.linear(y, _t(w, p + ".pointwise_conv2.weight")[:, :, 0], _t(w, p + ".pointwise_conv2.bias"))


def block(w, i, x, pos, cfg: EncoderConfig):
    p = f"layers.{i}"
    x = x + 0.5 * _ff(w, p + ".feed_forward1", _ln(w, p + ".norm_feed_forward1", x))
    x = x + _attention(w, p + ".self_attn", _ln(w, p + ".norm_self_att", x), pos, cfg)
    x = x + _conv_module(w, p + ".conv", _ln(w, p + ".norm_conv", x), cfg)
    x = x + 0.5 * _ff(w, p + ".feed_forward2", _ln(w, p + ".norm_feed_forward2", x))
    return _ln(w, p + ".norm_out", x)


@torch.no_grad()
def encoder_forward(w: dict, feats: np.ndarray, cfg: EncoderConfig, return_intermediates: bool = False):
    """feats [T, mels] f32 -> [T', d_model] f32 (time-major)."""
    x = subsampling(w, torch.from_numpy(np.ascontiguousarray(feats, np.float32)), cfg)
    inter = {"subsampling": x.numpy().copy()} if return_intermediates else None
    pos = rel_positions(x.shape[0], cfg.d_model)
    for i in range(cfg.layers):
        x = block(w, i, x, pos, cfg)
        if return_intermediates:
            inter[f"layer{i}"] = x.numpy().copy()
    out = x.numpy()
    return (out, inter) if return_intermediates else out
