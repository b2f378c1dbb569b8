"""The encoder at full depth (24 Conformer blocks) against the fp32 CPU oracle, and how the error grows with depth.

Configuration 2 of the benchmark list: a batch of 32 clips x 1001 normalised mel frames (10 s clips of the seeded
sinusoid + noise distribution, through the GPU frontend), seeded N(0, 0.02) weights with identity norms, 126 encoder
frames per clip.  A d-block model is the first d blocks of the 24-block one (each block ends with its own closing
LayerNorm), so the oracle runs once at depth 24 and its per-block outputs serve every depth.

Tolerances (relative L2 error of the encoder output per clip): bf16 <= 2e-2; the FP8-e4m3 variant has the goal 5e-2.
The reference states looser bounds for its own backend comparison (dev-tools/python/compare_coreml.py:37-41:
max-abs 2e-1 on the encoder output).

The measured tables are written as markdown files into $SB_REPORT_DIR when that variable is set.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import encoder_oracle as eo
from scriptrs_b200 import synth

BF16_TOL = 2e-2
FP8_GOAL = 5e-2
DEPTHS = (1, 2, 4, 8, 16, 24)
CHECKED = (0, 7, 19, 31)  # clips of the batch compared with the oracle
FP8_MASKS = {1: "ff up", 2: "ff down", 4: "qkv", 8: "conv pw1", 3: "ff up+down", 12: "qkv+pw1", 15: "all four"}


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b.astype(np.float64)))


@pytest.fixture(scope="module")
def config2(ctx):
    """Features of the 32-clip batch (GPU frontend) + one 1497-frame long-form clip, and the oracle's per-block
    outputs for the checked clips."""
    import scriptrs_b200 as sb

    clips = [synth.clip_audio(160000, 500 + i) for i in range(32)] + [synth.clip_audio(239360, 900)]
    feats = sb.ParakeetFeatureExtractor(ctx).extract_batch(clips)
    assert feats[0].shape == (1001, 128) and feats[32].shape == (1497, 128)
    w = synth.seeded_model(24)
    cfg = eo.EncoderConfig(layers=24)
    checked = list(CHECKED) + [32]
    oracle = {}
    for i in checked:
        _, inter = eo.encoder_forward(w, feats[i], cfg, return_intermediates=True)
        oracle[i] = {d: inter[f"layer{d - 1}"] for d in DEPTHS}
    return dict(feats=feats, w=w, oracle=oracle, checked=checked)


def encode(ctx, feats_list):
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


def write_report(name, lines):
    d = os.environ.get("SB_REPORT_DIR")
    if d:
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, name), "w") as f:
            f.write("\n".join(lines) + "\n")


def test_config2_bf16_parity_at_every_depth(ctx, config2):
    import scriptrs_b200 as sb

    feats, w, oracle, checked = config2["feats"], config2["w"], config2["oracle"], config2["checked"]
    rows = {}
    for d in DEPTHS:
        sb.load_model(ctx, w, encoder_layers=d, has_encoder=True)
        got = encode(ctx, feats)
        assert got[0].shape == (126, 1024) and got[32].shape == (188, 1024)
        assert all(np.isfinite(g).all() for g in got)
        rows[d] = [rel(got[i], oracle[i][d]) for i in checked]
    lines = ["| depth | " + " | ".join(f"clip {i}" + (" (1497 frames)" if i == 32 else "") for i in checked) + " |",
             "|---|" + "---|" * len(checked)]
    lines += [f"| {d} | " + " | ".join(f"{e:.2e}" for e in rows[d]) + " |" for d in DEPTHS]
    write_report("encoder_error_vs_depth_bf16.md", lines)
    worst = {d: max(rows[d]) for d in DEPTHS}
    assert all(worst[d] <= BF16_TOL for d in DEPTHS), "relative L2 error per depth: " + str(worst)


def test_fp8_error_per_gemm_kind_and_depth(ctx, config2):
    """The ablation behind the FP8 default: error against the fp32 oracle for each group of GEMMs switched to e4m3
    (option fp8_mask: 1 ff up, 2 ff down, 4 QKV, 8 first pointwise), with the hidden row of the feed-forward
    module quantised by its advance bound or by its true maximum (option fp8_hidden_amax), at depths 1, 4 and 24.
    Asserts only that every variant stays finite and within 2.5x the goal; the goal itself is asserted in the
    two tests below."""
    import scriptrs_b200 as sb

    feats, w, oracle = config2["feats"], config2["w"], config2["oracle"]
    sub = [feats[i] for i in CHECKED]
    lines = ["| depth | fp8_mask | GEMMs in e4m3 | hidden-row scale | worst rel. L2 error of 4 clips |", "|---|---|---|---|---|"]
    worst_all = 0.0
    for d in (1, 4, 24):
        sb.load_model(ctx, w, encoder_layers=d, has_encoder=True, fp8_weights=True)
        ctx.set_option("fp8", 1)
        try:
            for mask, what in FP8_MASKS.items():
                for amax in ((0, 1) if (mask & 3) == 3 else (0,)):
                    ctx.set_option("fp8_mask", mask)
                    ctx.set_option("fp8_hidden_amax", amax)
                    got = encode(ctx, sub)
                    assert all(np.isfinite(g).all() for g in got)
                    e = max(rel(g, oracle[i][d]) for g, i in zip(got, CHECKED))
                    worst_all = max(worst_all, e)
                    scale = "-" if (mask & 3) != 3 else ("true row maximum" if amax else "advance bound")
                    lines.append(f"| {d} | {mask} | {what} | {scale} | {e:.2e} |")
        finally:
            ctx.set_option("fp8_mask", 8)
            ctx.set_option("fp8_hidden_amax", 0)
            ctx.set_option("fp8", 0)
    write_report("encoder_error_fp8_ablation.md", lines)
    assert worst_all <= 2.5 * FP8_GOAL, "\n".join(lines)


def fp8_error_at_24(ctx, config2, mask):
    import scriptrs_b200 as sb

    sb.load_model(ctx, config2["w"], encoder_layers=24, has_encoder=True, fp8_weights=True)
    ctx.set_option("fp8", 1)
    ctx.set_option("fp8_mask", mask)
    try:
        got = encode(ctx, [config2["feats"][i] for i in CHECKED])
    finally:
        ctx.set_option("fp8_mask", 8)
        ctx.set_option("fp8", 0)
    return max(rel(g, config2["oracle"][i][24]) for g, i in zip(got, CHECKED))


def test_fp8_default_subset_meets_goal_at_24_blocks(ctx, config2):
    """The library's default FP8 configuration (fp8_mask = 8) on configuration 2."""
    e = fp8_error_at_24(ctx, config2, 8)
    assert e <= FP8_GOAL, e


@pytest.mark.xfail(strict=True, reason="goal missed: all four GEMM groups in e4m3 give 1.0e-1 at 24 blocks with N(0, 0.02) "
                                       "random weights (goal 5e-2); test_fp8_error_per_gemm_kind_and_depth records the ablation")
def test_fp8_all_gemm_groups_meet_goal_at_24_blocks(ctx, config2):
    e = fp8_error_at_24(ctx, config2, 15)
    assert e <= FP8_GOAL, e
