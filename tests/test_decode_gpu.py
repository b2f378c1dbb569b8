"""Batched TDT greedy decode on the GPU (through the C ABI) against the CPU oracle.

Bit-exactness: the token ids, frame indices and durations the GPU emits must equal what the
reference's state machine produces when it is fed the very logits the GPU computed (logit replay).
Numerics: the GPU's logits (fp32 CUDA-core path, and the three-term split-bf16 tensor-core path) must agree with
the fp32 oracle's to 1e-4 relative."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

import oracle


def decode_gpu(ctx, encs, trace=True):
    import scriptrs_b200 as sb

    offs = np.zeros(len(encs) + 1, np.int64)
    offs[1:] = np.cumsum([e.shape[0] for e in encs])
    cat = np.concatenate([e for e in encs if e.shape[0]] or [np.zeros((0, 1024), np.float32)])
    d_enc = torch.from_numpy(np.ascontiguousarray(cat)).cuda() if cat.size else torch.zeros(1, 1024, device="cuda")
    torch.cuda.synchronize()
    tmax = int(max(e.shape[0] for e in encs))
    return sb.tdt_decode_device(ctx, d_enc.data_ptr(), offs, trace_cap=(11 * tmax + 2) if trace else 0)


@pytest.fixture(params=["tensor", "simt"], autouse=True)
def decode_path(request, ctx):
    """Every test runs on both decoders: split-bf16 tensor-core steps (default) and the fp32 persistent kernel."""
    ctx.set_option("simt_decode", 1 if request.param == "simt" else 0)
    yield request.param
    ctx.set_option("simt_decode", 0)


@pytest.fixture(scope="module")
def weights(ctx):
    import scriptrs_b200 as sb

    wn = oracle.seeded_decoder_weights(7)
    sb.load_model(ctx, wn, encoder_layers=0, has_encoder=False, has_decoder=True)
    return wn


def test_config3_replay_is_bit_exact_and_logits_match(ctx, weights):
    rng = np.random.default_rng(33)
    encs = [rng.standard_normal((126, 1024)).astype(np.float32) for _ in range(32)]
    got = decode_gpu(ctx, encs)
    w = oracle.tdt_weights_from_named(weights)
    identical = 0
    for g, enc in zip(got, encs):
        rep = oracle.greedy_replay(g["logits"], time_steps=126)
        assert rep["steps"] == g["steps"]
        assert np.array_equal(rep["tokens"], g["tokens"])
        assert np.array_equal(rep["frames"], g["frames"])
        assert np.array_equal(rep["durations"], g["durations"])
        assert np.allclose(rep["conf"], g["conf"], rtol=1e-5, atol=1e-7)
        full = oracle.tdt_decode(w, enc, want_trace=True)
        # first iteration: same inputs on both sides, so the logits must agree numerically
        a, b = g["logits"][0], full["logits"][0]
        assert np.linalg.norm(a - b) / np.linalg.norm(b) < 1e-4
        if (len(full["tokens"]) == len(g["tokens"]) and np.array_equal(full["tokens"], g["tokens"])
                and np.array_equal(full["frames"], g["frames"]) and np.array_equal(full["durations"], g["durations"])):
            identical += 1
            n = min(len(g["logits"]), len(full["logits"]))
            assert np.abs(g["logits"][:n] - full["logits"][:n]).max() < 5e-4
    # an fp32 near-tie may flip a decision between two summation orders; it must be rare
    assert identical >= 30, identical


def test_ragged_batch_and_edge_lengths(ctx, weights):
    rng = np.random.default_rng(5)
    lens = [1, 2, 7, 0, 188, 33, 167, 1]
    encs = [rng.standard_normal((t, 1024)).astype(np.float32) for t in lens]
    got = decode_gpu(ctx, encs)
    for g, t in zip(got, lens):
        if t == 0:
            assert g["steps"] == 0 and len(g["tokens"]) == 0
            continue
        rep = oracle.greedy_replay(g["logits"], time_steps=t)
        assert rep["steps"] == g["steps"]
        for k in ("tokens", "frames", "durations"):
            assert np.array_equal(rep[k], g[k])
        assert (g["frames"] < t).all()


def test_results_do_not_depend_on_batch_composition(ctx, weights):
    rng = np.random.default_rng(9)
    a = rng.standard_normal((60, 1024)).astype(np.float32)
    b = rng.standard_normal((90, 1024)).astype(np.float32)
    alone = decode_gpu(ctx, [a], trace=False)[0]
    mixed = decode_gpu(ctx, [b, a, b, b], trace=False)
    for k in ("tokens", "frames", "durations", "conf"):
        assert np.array_equal(alone[k], mixed[1][k])
        assert np.array_equal(mixed[0][k], mixed[2][k])


def test_max_tokens_overflow_is_reported(ctx, weights):
    import scriptrs_b200 as sb

    enc = torch.randn(50, 1024, device="cuda")
    torch.cuda.synchronize()
    with pytest.raises(sb.ScriptrsError) as e:
        sb.tdt_decode_device(ctx, enc.data_ptr(), np.array([0, 50], np.int64), max_tokens=2)
    assert e.value.status == 12


def test_many_sequences_span_several_gemm_tiles(ctx, weights, decode_path):
    """300 ragged sequences: more than two 128-row tiles of the tensor-core products, and the wide-tile launch
    of the fp32 kernel; every sequence must equal its own replay and what it gives when decoded alone."""
    rng = np.random.default_rng(77)
    lens = rng.integers(1, 40, size=300)
    encs = [rng.standard_normal((int(t), 1024)).astype(np.float32) for t in lens]
    got = decode_gpu(ctx, encs)
    for g, t in zip(got, lens):
        rep = oracle.greedy_replay(g["logits"], time_steps=int(t))
        assert rep["steps"] == g["steps"]
        for k in ("tokens", "frames", "durations"):
            assert np.array_equal(rep[k], g[k])
    for i in (0, 131, 299):
        alone = decode_gpu(ctx, [encs[i]], trace=False)[0]
        for k in ("tokens", "frames", "durations", "conf"):
            assert np.array_equal(alone[k], got[i][k])
