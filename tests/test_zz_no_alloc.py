"""sb_frontend_device_noalloc, the frontend entry point for callers that cannot allocate device memory
(an ingest thread that must not trigger cudaMalloc's device-wide synchronisation while other streams
run, or a host whose own pool owns all device memory).  It keeps its scratch in a fixed device array
inside the library, so the checks are: same features as the allocating entry point, bit for bit, on
two calls in a row (the second smaller, so stale scratch from the first must not matter), a batch that
fills the fixed capacity exactly, free device memory unchanged across calls (the property in the name),
and clear refusals beyond the capacity and on a capturing stream.  Collected last on purpose."""
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


def test_full_capacity_batch_and_no_device_allocation(ctx):
    """1024 short clips fill the last rows of the fixed metadata and statistics regions; the result must still
    equal the allocating entry point bit for bit, and the free device memory that the driver reports must not
    move across the calls (the first call on the device has already happened in the tests above or happens here
    before the measurement)."""
    import scriptrs_b200 as sb

    lens = [300 + (7 * i) % 500 for i in range(1024)]
    clips = [synth.clip_audio(n, 3000 + i) if i % 9 else np.zeros(n, np.float32) for i, n in enumerate(lens)]
    offs = np.zeros(1025, np.int64)
    offs[1:] = np.cumsum(lens)
    pcm = torch.from_numpy(np.concatenate(clips)).cuda()
    rows = sum(sb.num_frames(n) for n in lens)
    ref = torch.full((rows, 128), float("nan"), device="cuda")
    got = torch.full((rows, 128), float("nan"), device="cuda")
    sb.ParakeetFeatureExtractor(ctx).extract_device(pcm.data_ptr(), offs, ref.data_ptr())
    ctx.synchronize()
    sb.frontend_device_noalloc(pcm.data_ptr(), offs, got.data_ptr())   # first call on the device at the latest
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        got.fill_(float("nan"))
        sb.frontend_device_noalloc(pcm.data_ptr(), offs, got.data_ptr())
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0
        assert torch.equal(ref, got)


def test_call_on_a_capturing_stream_is_refused(ctx):
    import scriptrs_b200 as sb

    clip = synth.clip_audio(16000, 6)
    pcm = torch.from_numpy(clip).cuda()
    offs = np.array([0, clip.size], np.int64)
    out = torch.empty(sb.num_frames(clip.size), 128, device="cuda")
    sb.frontend_device_noalloc(pcm.data_ptr(), offs, out.data_ptr())
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        graph.capture_begin(capture_error_mode="thread_local")
        try:
            with pytest.raises(sb.ScriptrsError) as e:
                sb.frontend_device_noalloc(pcm.data_ptr(), offs, out.data_ptr(), stream=stream.cuda_stream)
            out.zero_()  # the capture records at least one node
        finally:
            graph.capture_end()
    assert e.value.status == 11 and "capture" in e.value.message
    # and the entry point still works afterwards
    sb.frontend_device_noalloc(pcm.data_ptr(), offs, out.data_ptr())
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
