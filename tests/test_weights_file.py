"""Weight files (safetensors layout) read by sb_model_load_file: the stand-in for the reference's bundle directory
(ModelBundle::from_dir / validate_base, src/models.rs:31-104; its own tests src/models.rs:251-340 use tempfile
directories the same way)."""
import json
import os
import struct

import numpy as np
import pytest

import scriptrs_b200 as sb
from scriptrs_b200 import synth, weights


def test_header_listing_round_trip(tmp_path):
    t = {"a.weight": np.arange(12, dtype=np.float32).reshape(3, 4), "b": np.float32(2.5).reshape(()),
         "layers.0.x": np.ones((2, 1, 3), np.float32), "tricky \"name\"é": np.zeros(5, np.float32)}
    for dt in ("F32", "F16", "BF16"):
        p = str(tmp_path / f"w_{dt}.safetensors")
        weights.save_safetensors(p, t, dtype=dt, metadata={"format": "pt", "note": "x"})
        got = {n: (d, s) for n, d, s in weights.list_weights_file(p)}
        assert got == {n: (dt, tuple(np.asarray(a).shape)) for n, a in t.items()}


def test_missing_file_is_a_missing_model_asset(tmp_path):
    with pytest.raises(sb.ScriptrsError) as e:
        weights.list_weights_file(str(tmp_path / "nope" / "model.safetensors"))
    assert e.value.status == 3 and "model.safetensors" in e.value.message      # MissingModelAsset { path }
    with pytest.raises(sb.ScriptrsError) as e:
        weights.validate_bundle(str(tmp_path))
    assert e.value.status == 3 and "parakeet-v2" in e.value.message


@pytest.mark.parametrize("damage", ["short", "header_len", "json", "range", "dtype", "no_shape"])
def test_malformed_files_are_io_errors(tmp_path, damage):
    p = str(tmp_path / "bad.safetensors")
    hdr = {"x": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}
    data = b"\0" * 16
    if damage == "range":
        hdr["x"]["data_offsets"] = [0, 32]
    if damage == "dtype":
        hdr["x"]["dtype"] = "I64"
    if damage == "no_shape":
        del hdr["x"]["shape"]
    h = json.dumps(hdr).encode()
    if damage == "json":
        h = h[:-3]
    blob = struct.pack("<Q", len(h)) + h + data
    if damage == "short":
        blob = blob[:5]
    if damage == "header_len":
        blob = struct.pack("<Q", 1 << 40) + h + data
    with open(p, "wb") as f:
        f.write(blob)
    with pytest.raises(sb.ScriptrsError) as e:
        weights.list_weights_file(p)
    assert e.value.status == 4, e.value


@pytest.mark.gpu
def test_model_from_file_equals_model_from_memory(ctx, tmp_path):
    """The seeded weights through a file (f32, behind a name prefix, block count taken from the file) must give the
    encoder and decoder outputs of the same weights handed over in memory, bit for bit; a bf16 file the outputs of
    the weights rounded to bf16 first."""
    torch = pytest.importorskip("torch")
    w = synth.seeded_model(2)
    feats = np.random.default_rng(0).standard_normal((700, 128)).astype(np.float32)

    def run():
        d_feats = torch.from_numpy(feats).cuda()
        d_out = torch.empty(sb.encoder_num_frames(700), 1024, device="cuda")
        torch.cuda.synchronize()
        eo = sb.encode_device(ctx, d_feats.data_ptr(), np.array([0, 700], np.int64), d_out.data_ptr())
        ctx.synchronize()
        dec = sb.tdt_decode_device(ctx, d_out.data_ptr(), eo)[0]
        return d_out.cpu().numpy(), dec["tokens"]

    sb.load_model(ctx, w, encoder_layers=2, has_encoder=True, has_decoder=True)
    ref_enc, ref_tok = run()
    p = str(tmp_path / "parakeet-v2" / "model.safetensors")
    weights.save_safetensors(p, {"model." + k: v for k, v in w.items()} | {"other.tensor": np.zeros(3, np.float32)})
    weights.load_model_file(ctx, p, prefix="model.")
    enc, tok = run()
    assert np.array_equal(enc, ref_enc) and np.array_equal(tok, ref_tok)

    def bf16(a):
        u = np.ascontiguousarray(a, np.float32).view(np.uint32)
        return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32).reshape(a.shape)

    weights.save_safetensors(p, w, dtype="BF16")
    weights.load_model_file(ctx, p, encoder_layers=2)
    enc_b, _ = run()
    sb.load_model(ctx, {k: bf16(v) for k, v in w.items()}, encoder_layers=2, has_encoder=True, has_decoder=True)
    enc_r, _ = run()
    assert np.array_equal(enc_b, enc_r)
    # a tensor missing from the file is reported by name, as a missing asset
    short = dict(w)
    del short["joint.out.bias"]
    weights.save_safetensors(p, short)
    with pytest.raises(sb.ScriptrsError) as e:
        weights.load_model_file(ctx, p)
    assert e.value.status == 3 and "joint.out.bias" in e.value.message


@pytest.mark.gpu
def test_pipeline_from_dir(ctx, tmp_path):
    """TranscriptionPipeline::from_dir (src/pipeline.rs:35-46) over a bundle directory written here."""
    w = synth.seeded_model(1)
    root = str(tmp_path)
    weights.save_safetensors(os.path.join(root, weights.MODEL_FILE), w)
    with pytest.raises(sb.ScriptrsError) as e:                      # vocabulary still missing
        sb.TranscriptionPipeline.from_dir(root, ctx=ctx)
    assert e.value.status == 3 and "vocab.txt" in e.value.message
    with open(os.path.join(root, weights.VOCAB_FILE), "w", encoding="utf-8") as f:
        f.write("".join(f"▁t{i} {i}\n" for i in range(1024)) + "<blk> 1024\n")
    pipe = sb.TranscriptionPipeline.from_dir(root, ctx=ctx)
    res = pipe.run(synth.clip_audio(64000, 1))
    assert res.duration_seconds == 4.0
    sb.load_model(ctx, w, encoder_layers=1, has_encoder=True, has_decoder=True)
    ref = sb.TranscriptionPipeline(ctx, pipe.vocab).run(synth.clip_audio(64000, 1))
    assert res.text == ref.text and res.tokens == ref.tokens


@pytest.mark.gpu
def test_long_form_from_dir_loads_the_vad_file_if_present(tmp_path):
    """LongFormTranscriptionPipeline::from_dir + load_vad (src/long_form.rs:100-123,663-670): the VAD network is
    optional at construction and only needed by the Vad mode; its file (public Silero state-dict names behind
    "_model.", here as bf16) gives the probabilities of the same weights loaded from memory."""
    root = str(tmp_path)
    weights.save_safetensors(os.path.join(root, weights.MODEL_FILE), synth.seeded_model(1))
    with open(os.path.join(root, weights.VOCAB_FILE), "w", encoding="utf-8") as f:
        f.write("".join(f"▁t{i} {i}\n" for i in range(1024)) + "<blk> 1024\n")
    audio = synth.sparse_speech_audio(16000 * 40, 12)
    lf = sb.LongFormTranscriptionPipeline.from_dir(root)
    try:
        assert lf.vad is None
        with pytest.raises(sb.ScriptrsError) as e:
            lf.run_with_config(audio, sb.LongFormConfig(mode=sb.LongFormMode.Vad))
        assert e.value.status == 3
        assert len(lf.run(audio).chunks) <= 1                      # the Fast mode needs no VAD network
        with pytest.raises(sb.ScriptrsError) as e:
            weights.validate_with_vad(root)
        assert e.value.status == 3 and "silero-vad" in e.value.message
    finally:
        lf.inner.ctx.close()
    vw = synth.energy_vad_weights()
    weights.save_safetensors(weights.vad_path(root), {"_model." + k: v for k, v in vw.items()})
    assert weights.validate_with_vad(root)[2].endswith("silero-vad.safetensors")
    lf = sb.LongFormTranscriptionPipeline.from_dir(root)
    try:
        assert lf.vad is not None
        from_file = lf.vad.process(audio)
        res = lf.run_with_config(audio, sb.LongFormConfig(mode=sb.LongFormMode.Vad))
        assert len(res.chunks) >= 1
        from_memory = sb.SileroVad(lf.inner.ctx, vw).process(audio)
        assert np.array_equal(from_file, from_memory)
    finally:
        lf.inner.ctx.close()
