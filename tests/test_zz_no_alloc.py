"""sb_frontend_device_noalloc, the frontend entry point for callers that cannot allocate device memory
(an ingest thread that must not trigger cudaMalloc's device-wide synchronisation while other streams
run, or a host whose own pool owns all device memory).  It keeps its scratch in a fixed device array
inside the library, so the checks are: same features as the allocating entry point, bit for bit, on
two calls in a row (the second smaller, so stale scratch from the first must not matter), and a clear
refusal beyond the fixed capacity.  Collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from scriptrs_b200 import synth


def run_both(ctx, clips):
    import scriptrs_b200 as sb

    offs = np.zeros(len(clips) + 1, np.int64)
    offs[1:] = np.cumsum([c.size for c in clips])
    pcm = torch.from_numpy(np.concatenate(clips)).cuda()
    rows = sum(sb.num_frames(c.size) for c in clips)
    ref = torch.full((rows, 128), float("nan"), device="cuda")
    got = torch.full((rows, 128), float("nan"), device="cuda")
    torch.cuda.synchronize()
    fo_ref = sb.ParakeetFeatureExtractor(ctx).extract_device(pcm.data_ptr(), offs, ref.data_ptr())
    ctx.synchronize()
    stream = torch.cuda.Stream()
    fo_got = sb.frontend_device_noalloc(pcm.data_ptr(), offs, got.data_ptr(), stream=stream.cuda_stream)
    stream.synchronize()
    return fo_ref, fo_got, ref.cpu().numpy(), got.cpu().numpy()


def test_two_calls_in_a_row_match_the_allocating_entry_point(ctx):
    first = [synth.clip_audio(n, 40 + i) for i, n in enumerate((48000, 239360, 16000, 5121))] + [np.zeros(32000, np.float32)]
    second = [synth.clip_audio(20000, 77), np.zeros(48000, np.float32)]
    for clips in (first, second):
        fo_ref, fo_got, ref, got = run_both(ctx, clips)
        assert np.array_equal(fo_ref, fo_got)
        assert not np.isnan(got).any()
        assert np.array_equal(ref, got)   # identical kernels and inputs: tolerance zero


def test_unnormalised_output_and_capacity_limit(ctx):
    import scriptrs_b200 as sb

    clip = synth.clip_audio(32000, 5)
    pcm = torch.from_numpy(clip).cuda()
    offs = np.array([0, clip.size], np.int64)
    a = torch.empty(sb.num_frames(clip.size), 128, device="cuda")
    b = torch.empty_like(a)
    torch.cuda.synchronize()
    sb.ParakeetFeatureExtractor(ctx).extract_device(pcm.data_ptr(), offs, a.data_ptr(), normalize=False)
    ctx.synchronize()
    sb.frontend_device_noalloc(pcm.data_ptr(), offs, b.data_ptr(), normalize=False)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    too_many = np.arange(1026, dtype=np.int64) * 16
    with pytest.raises(sb.ScriptrsError) as e:
        sb.frontend_device_noalloc(pcm.data_ptr(), too_many, b.data_ptr())
    assert e.value.status == 11 and "1024" in e.value.message
