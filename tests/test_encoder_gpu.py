"""CUDA FastConformer encoder (through the C ABI) against the fp32 CPU oracle, same seeded weights.

Tolerance: relative L2 error <= 2e-2 on the encoder output for the bf16 path."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import encoder_oracle as eo

BF16_TOL = 2e-2


def run_gpu(ctx, feats_list):
    import scriptrs_b200 as sb

    fo = np.zeros(len(feats_list) + 1, np.int64)
    fo[1:] = np.cumsum([f.shape[0] for f in feats_list])
    d_feats = torch.from_numpy(np.concatenate(feats_list)).cuda()
    n_out = sum(sb.encoder_num_frames(f.shape[0]) for f in feats_list)
    d_out = torch.full((n_out, 1024), float("nan"), device="cuda")
    torch.cuda.synchronize()
    offs = sb.encode_device(ctx, d_feats.data_ptr(), fo, d_out.data_ptr())
    ctx.synchronize()
    out = d_out.cpu().numpy()
    return [out[offs[i]:offs[i + 1]] for i in range(len(feats_list))]


@pytest.fixture(params=["tensor-core attention", "simt attention"])
def attention_mode(ctx, request):
    ctx.set_option("simt_attention", int(request.param.startswith("simt")))
    yield request.param
    ctx.set_option("simt_attention", 0)


@pytest.mark.parametrize("layers", [0, 1, 2])
def test_shallow_stacks_match_oracle(ctx, layers, attention_mode):
    import scriptrs_b200 as sb

    if layers == 0 and attention_mode.startswith("simt"):
        pytest.skip("no attention in a 0-block stack")
    cfg = eo.EncoderConfig(layers=layers)
    w = eo.seeded_weights(cfg, seed=11, std=0.02, plain_norms=False)
    sb.load_model(ctx, w, encoder_layers=layers)
    rng = np.random.default_rng(layers)
    feats = [rng.standard_normal((t, 128)).astype(np.float32) for t in (203, 1001, 9, 64, 1497, 1, 1024, 1030, 1329)]
    got = run_gpu(ctx, feats)
    for f, g in zip(feats, got):
        r = eo.encoder_forward(w, f, cfg)
        assert g.shape == r.shape == (eo.subsampled_length(f.shape[0]), 1024)
        assert np.isfinite(g).all()
        err = np.linalg.norm(g - r) / np.linalg.norm(r)
        assert err <= BF16_TOL, (layers, f.shape[0], err)


def test_scale_input_and_batch_independence(ctx):
    import scriptrs_b200 as sb

    cfg = eo.EncoderConfig(layers=1, scale_input=True)
    w = eo.seeded_weights(cfg, seed=12, std=0.02, plain_norms=False)
    sb.load_model(ctx, w, encoder_layers=1, scale_input=True)
    rng = np.random.default_rng(5)
    a = rng.standard_normal((333, 128)).astype(np.float32)
    b = rng.standard_normal((120, 128)).astype(np.float32)
    alone = run_gpu(ctx, [a])[0]
    together = run_gpu(ctx, [b, a, b])
    assert np.array_equal(alone, together[1])       # a clip's result does not depend on its neighbours
    assert np.array_equal(together[0], together[2])
    r = eo.encoder_forward(w, a, cfg)
    assert np.linalg.norm(alone - r) / np.linalg.norm(r) <= BF16_TOL


def test_missing_tensor_is_reported(ctx):
    import scriptrs_b200 as sb

    cfg = eo.EncoderConfig(layers=1)
    w = eo.seeded_weights(cfg, seed=1)
    del w["layers.0.conv.norm.running_var"]
    with pytest.raises(sb.ScriptrsError) as e:
        sb.load_model(ctx, w, encoder_layers=1)
    assert e.value.status == 3 and "running_var" in e.value.message


def test_too_many_feature_frames_is_rejected(ctx):
    import scriptrs_b200 as sb

    cfg = eo.EncoderConfig(layers=0)
    sb.load_model(ctx, eo.seeded_weights(cfg, seed=1), encoder_layers=0)
    d = torch.zeros(1502, 128, device="cuda")
    o = torch.zeros(200, 1024, device="cuda")
    with pytest.raises(sb.ScriptrsError) as e:
        sb.encode_device(ctx, d.data_ptr(), np.array([0, 1502], np.int64), o.data_ptr())
    assert e.value.status == 6


# The stated goal for the FP8 variant is 5e-2 relative L2 error against the fp32 oracle.  With the seeded random
# weights only the first pointwise convolution of the convolution module can run in e4m3 within that goal (the
# library's default fp8_mask = 8); each of the other GEMM groups alone already exceeds it at depth, so the all-groups variant is an expected failure below,
# asserted against the goal itself and not against a loosened bound.
FP8_GOAL = 5e-2


def fp8_errors(ctx, layers, mask):
    import scriptrs_b200 as sb

    cfg = eo.EncoderConfig(layers=layers)
    w = eo.seeded_weights(cfg, seed=31, std=0.02, plain_norms=False)
    sb.load_model(ctx, w, encoder_layers=layers, fp8_weights=True)
    rng = np.random.default_rng(layers)
    feats = [rng.standard_normal((t, 128)).astype(np.float32) for t in (1001, 203, 1497, 9)]
    ctx.set_option("fp8", 1)
    if mask is not None:
        ctx.set_option("fp8_mask", mask)
    try:
        got = run_gpu(ctx, feats)
    finally:
        ctx.set_option("fp8_mask", 8)
        ctx.set_option("fp8", 0)
    bf = run_gpu(ctx, feats)
    out = []
    for f, g, b in zip(feats, got, bf):
        r = eo.encoder_forward(w, f, cfg)
        assert np.isfinite(g).all()
        assert np.linalg.norm(b - r) / np.linalg.norm(r) <= BF16_TOL
        assert not np.array_equal(g, b)  # the switch really changes the arithmetic
        out.append(float(np.linalg.norm(g - r) / np.linalg.norm(r)))
    return out


@pytest.mark.parametrize("layers", [1, 2, 4])
def test_fp8_default_subset_meets_goal(ctx, layers):
    """The default FP8 configuration (fp8_mask = 8: first pointwise convolution in e4m3) against the fp32 oracle."""
    errs = fp8_errors(ctx, layers, None)
    assert max(errs) <= FP8_GOAL, (layers, errs)


@pytest.mark.xfail(strict=True, reason="goal missed: feed-forward, QKV and pointwise GEMMs all in e4m3 give 7.2e-2 at 4 "
                                       "blocks and 1.0e-1 at 24 with N(0, 0.02) random weights (goal 5e-2)")
def test_fp8_all_gemm_groups_meet_goal(ctx):
    errs = fp8_errors(ctx, 4, 15)
    assert max(errs) <= FP8_GOAL, errs


def test_fp8_needs_fp8_weights(ctx):
    import scriptrs_b200 as sb

    cfg = eo.EncoderConfig(layers=1)
    sb.load_model(ctx, eo.seeded_weights(cfg, seed=1), encoder_layers=1)
    with pytest.raises(sb.ScriptrsError) as e:
        ctx.set_option("fp8", 1)
    assert e.value.status == 3


def test_large_batch_reaches_two_cta_tiles_and_matches_single_cta_and_oracle(ctx):
    """48 clips x 188 frames = 9024 rows: enough 256 x 256 tiles for the products to run on two-CTA clusters.
    The two tile shapes add the same products in the same order, so the outputs must be bit-identical; three of
    the clips are also checked against the oracle."""
    import scriptrs_b200 as sb

    cfg = eo.EncoderConfig(layers=1)
    w = eo.seeded_weights(cfg, seed=13, std=0.02, plain_norms=False)
    sb.load_model(ctx, w, encoder_layers=1)
    rng = np.random.default_rng(5)
    feats = [rng.standard_normal((1497 if i % 5 else 1201, 128)).astype(np.float32) for i in range(48)]
    try:
        ctx.set_option("gemm_pair_tiles", 0)
        single = run_gpu(ctx, feats)
        ctx.set_option("gemm_pair_tiles", 2)
        pair = run_gpu(ctx, feats)
    finally:
        ctx.set_option("gemm_pair_tiles", 1)
    default = run_gpu(ctx, feats)
    for a, b, c in zip(single, pair, default):
        assert np.array_equal(a, b) and np.array_equal(a, c)
    for i in (0, 5, 47):
        r = eo.encoder_forward(w, feats[i], cfg)
        err = np.linalg.norm(pair[i] - r) / np.linalg.norm(r)
        assert err <= BF16_TOL, (i, err)


def test_subsampling_tensor_core_kernel_against_cuda_core_kernel_and_oracle(ctx):
    """The first two sub-sampling stages run as an fp16 tensor-core product + packed-fp16 depthwise stage; the fp32
    CUDA-core kernel of the same stages (option simt_subsample) and the fp32 oracle are the checks.  0-block stack:
    the encoder output is the sub-sampling output."""
    import scriptrs_b200 as sb

    cfg = eo.EncoderConfig(layers=0)
    w = eo.seeded_weights(cfg, seed=17, std=0.05, plain_norms=False)
    sb.load_model(ctx, w, encoder_layers=0)
    rng = np.random.default_rng(9)
    feats = [(rng.standard_normal((t, 128)) * s).astype(np.float32) for t, s in
             ((1497, 1.0), (1, 1.0), (2, 3.0), (5, 1.0), (9, 0.1), (1001, 2.0), (333, 1.0), (8, 1.0), (1329, 1.0))]
    tc = run_gpu(ctx, feats)
    ctx.set_option("simt_subsample", 1)
    try:
        simt = run_gpu(ctx, feats)
    finally:
        ctx.set_option("simt_subsample", 0)
    for f, a, b in zip(feats, tc, simt):
        r = eo.encoder_forward(w, f, cfg)
        assert np.isfinite(a).all()
        assert np.linalg.norm(a - r) / np.linalg.norm(r) <= BF16_TOL, f.shape
        assert np.linalg.norm(b - r) / np.linalg.norm(r) <= BF16_TOL, f.shape
        assert np.linalg.norm(a - b) / np.linalg.norm(b) <= 1e-2, (f.shape, np.linalg.norm(a - b) / np.linalg.norm(b))
