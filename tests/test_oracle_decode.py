"""The decode oracle's state machine against hand-worked cases of the reference's loop
(src/model.rs:64-214; twin: dev-tools/python/compare_coreml.py:216-338)."""
import numpy as np

import oracle

V, D, BLANK = 1025, 5, 1024


def row(token, dur, tok_logit=5.0):
    r = np.zeros(V + D, np.float32)
    r[token] = tok_logit
    r[V + dur] = 3.0
    return r


def test_blank_with_zero_duration_advances_one_frame():
    lg = np.stack([row(BLANK, 0), row(BLANK, 0), row(BLANK, 0)])
    r = oracle.greedy_replay(lg, time_steps=3)
    assert r["steps"] == 3 and len(r["tokens"]) == 0
    assert list(r["step_frame"]) == [0, 1, 2]
    # the predictor runs once and its cache survives blanks (model.rs:150-152)
    assert list(r["step_ran_predictor"]) == [1, 0, 0]


def test_duration_jump_and_frame_recorded_before_advance():
    lg = np.stack([row(7, 2), row(9, 4)])
    r = oracle.greedy_replay(lg, time_steps=5)
    assert list(r["tokens"]) == [7, 9]
    assert list(r["frames"]) == [0, 2]          # model.rs:190-193
    assert list(r["durations"]) == [2, 4]
    assert r["steps"] == 2                      # the second jump overshoots T' = 5 and ends the loop
    assert list(r["step_ran_predictor"]) == [1, 1]


def test_at_most_ten_symbols_per_frame():
    lg = np.stack([row(3, 0)] * 10 + [row(BLANK, 0)])
    r = oracle.greedy_replay(lg, time_steps=2)
    # ten non-blank emissions with duration 0 stay on frame 0; the tenth forces the advance (model.rs:205)
    assert list(r["frames"]) == [0] * 10
    assert list(r["step_frame"]) == [0] * 10 + [1]
    assert r["steps"] == 11


def test_argmax_ties_go_to_the_lowest_index_and_confidence_is_max_softmax():
    r0 = np.zeros(V + D, np.float32)
    r0[5] = r0[9] = 2.0
    r0[V + 1] = r0[V + 3] = 1.0
    r = oracle.greedy_replay(r0[None], time_steps=1)
    assert list(r["tokens"]) == [5] and list(r["durations"]) == [1]
    e = np.exp(r0[:V] - r0[:V].max())
    assert abs(float(r["conf"][0]) - float(e.max() / e.sum())) < 1e-6


def test_full_decode_equals_replay_of_its_own_logits():
    w = oracle.tdt_weights_from_named(oracle.seeded_decoder_weights(3))
    enc = np.random.default_rng(0).standard_normal((20, 1024)).astype(np.float32)
    full = oracle.tdt_decode(w, enc, want_trace=True)
    rep = oracle.greedy_replay(full["logits"], time_steps=20)
    for k in ("tokens", "frames", "durations"):
        assert np.array_equal(full[k], rep[k])
    assert np.allclose(full["conf"], rep["conf"])
    assert full["steps"] == rep["steps"]


def test_lstm_matches_torch():
    torch = __import__("pytest").importorskip("torch")
    wn = oracle.seeded_decoder_weights(4)
    w = oracle.tdt_weights_from_named(wn)
    enc = np.random.default_rng(1).standard_normal((1, 1024)).astype(np.float32)
    full = oracle.tdt_decode(w, enc, want_trace=True)
    lstm = torch.nn.LSTM(640, 640, num_layers=2)
    sd = {}
    for l in range(2):
        sd[f"weight_ih_l{l}"] = torch.from_numpy(wn["predictor.lstm.weight_ih"][l])
        sd[f"weight_hh_l{l}"] = torch.from_numpy(wn["predictor.lstm.weight_hh"][l])
        sd[f"bias_ih_l{l}"] = torch.from_numpy(wn["predictor.lstm.bias_ih"][l])
        sd[f"bias_hh_l{l}"] = torch.from_numpy(wn["predictor.lstm.bias_hh"][l])
    lstm.load_state_dict(sd)
    with torch.no_grad():
        x = torch.from_numpy(wn["predictor.embedding"][1024])[None, None]
        dec, _ = lstm(x)
        z = torch.relu(torch.from_numpy(enc[0]) @ torch.from_numpy(wn["joint.enc.weight"]).T
                       + torch.from_numpy(wn["joint.enc.bias"])
                       + dec[0, 0] @ torch.from_numpy(wn["joint.pred.weight"]).T + torch.from_numpy(wn["joint.pred.bias"]))
        logits = z @ torch.from_numpy(wn["joint.out.weight"]).T + torch.from_numpy(wn["joint.out.bias"])
    assert np.allclose(full["logits"][0], logits.numpy(), atol=2e-5)
