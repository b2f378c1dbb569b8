"""Cross-checks the fp32 encoder oracle against the independent FastConformer implementation
that ships with `transformers` (same seeded weights loaded into both)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from oracle import encoder_oracle as eo


def hf_encoder(cfg, w):
    tr = pytest.importorskip("transformers")
    from transformers.models.parakeet.configuration_parakeet import ParakeetEncoderConfig
    from transformers.models.parakeet.modeling_parakeet import ParakeetEncoder

    hc = ParakeetEncoderConfig(hidden_size=cfg.d_model, num_hidden_layers=cfg.layers, num_attention_heads=cfg.heads,
                               intermediate_size=cfg.ff, conv_kernel_size=cfg.conv_kernel,
                               subsampling_conv_channels=cfg.sub_channels, num_mel_bins=cfg.mels,
                               scale_input=cfg.scale_input, dropout=0.0, layerdrop=0.0, activation_dropout=0.0,
                               attention_dropout=0.0, dropout_positions=0.0)
    hc._attn_implementation = "eager"
    m = ParakeetEncoder(hc).eval()
    sd = {k: torch.from_numpy(v) for k, v in w.items()}
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("num_batches_tracked" in k or "inv_freq" in k for k in missing), missing
    return m


@pytest.mark.parametrize("scale_input", [False, True])
def test_oracle_matches_transformers_parakeet_encoder(scale_input):
    cfg = eo.EncoderConfig(layers=2, d_model=64, heads=4, ff=128, conv_kernel=9, sub_channels=32, mels=128,
                           scale_input=scale_input)
    w = eo.seeded_weights(cfg, seed=3, std=0.1, plain_norms=False)
    rng = np.random.default_rng(0)
    feats = rng.standard_normal((203, 128)).astype(np.float32)
    mine = eo.encoder_forward(w, feats, cfg)
    m = hf_encoder(cfg, w)
    with torch.no_grad():
        ref = m(torch.from_numpy(feats)[None]).last_hidden_state[0].numpy()
    assert mine.shape == ref.shape == (eo.subsampled_length(203), 64)
    err = np.linalg.norm(mine - ref) / np.linalg.norm(ref)
    assert err < 1e-5, err


def test_per_clip_processing_equals_masked_padded_batch():
    cfg = eo.EncoderConfig(layers=1, d_model=64, heads=4, ff=128, sub_channels=32)
    w = eo.seeded_weights(cfg, seed=5, std=0.1, plain_norms=False)
    rng = np.random.default_rng(1)
    a = rng.standard_normal((160, 128)).astype(np.float32)
    b = rng.standard_normal((97, 128)).astype(np.float32)
    m = hf_encoder(cfg, w)
    batch = np.zeros((2, 160, 128), np.float32)
    batch[0] = a
    batch[1, :97] = b
    mask = torch.zeros(2, 160, dtype=torch.bool)
    mask[0] = True
    mask[1, :97] = True
    with torch.no_grad():
        ref = m(torch.from_numpy(batch), attention_mask=mask).last_hidden_state.numpy()
    tb = eo.subsampled_length(97)
    mine_b = eo.encoder_forward(w, b, cfg)
    err = np.linalg.norm(mine_b - ref[1, :tb]) / np.linalg.norm(ref[1, :tb])
    assert err < 1e-5, err


def test_subsampled_lengths():
    # 1501 -> 751 -> 376 -> 188 ; 1001 -> 126 ; 1497 -> 188 ; 1489 -> 187 ; 1329 -> 167
    for t, e in ((1501, 188), (1001, 126), (1497, 188), (1489, 187), (1329, 167), (1, 1), (8, 1), (9, 2)):
        assert eo.subsampled_length(t) == e
