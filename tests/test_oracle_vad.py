"""The numpy oracle of the voice-activity network against the same network written with torch's own layers
(F.pad reflect, F.conv1d, nn.LSTMCell): an independent implementation of every operator, fed the same seeded weights.
The reference keeps this network in a CoreML file outside its repository, so no golden output of it exists; what can be
pinned is that the oracle computes the public network shape the way a standard library does, window by window in the
streaming loop of src/long_form/vad.rs:61-98."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.nn.functional as F

from oracle import vad_oracle as vo
from scriptrs_b200 import synth


def torch_vad(weights, audio):
    w = {k: torch.from_numpy(np.ascontiguousarray(v, np.float32)) for k, v in weights.items()}
    cell = torch.nn.LSTMCell(128, 128)
    with torch.no_grad():
        cell.weight_ih.copy_(w["decoder.rnn.weight_ih"])
        cell.weight_hh.copy_(w["decoder.rnn.weight_hh"])
        cell.bias_ih.copy_(w["decoder.rnn.bias_ih"])
        cell.bias_hh.copy_(w["decoder.rnn.bias_hh"])
    h = torch.zeros(1, 128)
    c = torch.zeros(1, 128)
    context = torch.zeros(64)
    probs = []
    a = torch.from_numpy(np.asarray(audio, np.float32))
    with torch.no_grad():
        for start in range(0, a.numel(), 512):
            chunk = a[start:start + 512]
            if chunk.numel() < 512:                                   # vad.rs:82-85
                chunk = torch.cat([chunk, chunk[-1].repeat(512 - chunk.numel())])
            x = torch.cat([context, chunk])[None, None, :]            # [1, 1, 576], vad.rs:87-88
            x = F.pad(x, (0, 64), mode="reflect")
            y = F.conv1d(x, w["stft.forward_basis_buffer"], stride=128)            # [1, 258, 4]
            x = torch.sqrt(y[:, :129] ** 2 + y[:, 129:] ** 2)
            for i, stride in enumerate((1, 2, 2, 1)):
                x = F.relu(F.conv1d(x, w[f"encoder.{i}.reparam_conv.weight"], w[f"encoder.{i}.reparam_conv.bias"],
                                    stride=stride, padding=1))
            assert x.shape == (1, 128, 1)
            h, c = cell(x[:, :, 0], (h, c))
            out = torch.sigmoid(F.conv1d(F.relu(h)[:, :, None], w["decoder.decoder.2.weight"], w["decoder.decoder.2.bias"]))
            probs.append(float(out.mean()))
            context = chunk[-64:]                                     # vad.rs:95
    return np.array(probs, np.float32), h[0].numpy(), c[0].numpy()


@pytest.mark.parametrize("seed,n", [(5, 16000 * 12 + 77), (9, 513), (3, 64)])
def test_oracle_matches_torch_layers(seed, n):
    w = synth.seeded_vad_weights(seed)
    audio = synth.sparse_speech_audio(n, seed, speech_seconds=(0.5, 3.0), silence_seconds=(0.2, 1.0))
    want, h_t, c_t = torch_vad(w, audio)
    got, h, c = vo.vad_probabilities(w, audio, return_state=True)
    assert got.shape == want.shape == (-(-n // 512),)
    assert np.abs(got - want).max() < 2e-5
    assert np.abs(h - h_t).max() < 2e-5 and np.abs(c - c_t).max() < 2e-5


def test_energy_detector_weights_in_torch_layers():
    w = synth.energy_vad_weights()
    audio = synth.sparse_speech_audio(16000 * 10, 4)
    want, _, _ = torch_vad(w, audio)
    got = vo.vad_probabilities(w, audio)
    assert np.abs(got - want).max() < 2e-5
    assert (want > 0.95).any() and (want < 0.05).any()


def test_window_inputs_follow_the_streaming_loop():
    # vad.rs:78-95: 64 samples of context (zeros first), the last window filled with its last sample
    a = np.arange(1, 1030, dtype=np.float32)
    x = vo.vad_window_inputs(a)
    assert x.shape == (3, 576)
    assert np.all(x[0, :64] == 0) and np.array_equal(x[0, 64:], a[:512])
    assert np.array_equal(x[1, :64], a[448:512]) and np.array_equal(x[1, 64:], a[512:1024])
    assert np.array_equal(x[2, :64], a[960:1024]) and np.array_equal(x[2, 64:69], a[1024:1029])
    assert np.all(x[2, 69:] == a[-1])
