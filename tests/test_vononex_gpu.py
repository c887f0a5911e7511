"""The Vononex decoder on the GPU against the plain implementation (tests/plain/vononex_plain.py): every
mechanism's kernel alone, then whole models through the replay program's function (whole prompts, token by
token, portions down to two tokens, mixed batches with pages and slots used again), far keys made to stand
out, long decoding, and greedy generation through the engine's own entry point and scheduler."""
import copy
import math

import pytest
import torch

from helpers import run_trace_inprocess
from plain import vononex_plain as VP
from vononex_helpers import (CONFIG_P, CONFIG_Q, CONFIGS, TOLERANCE, VononexModel, compare, cut_steps, left, mingru,
                             mixed_steps, parallel, right, whole_steps)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
_models = {}


def _model(name, seed=5):
    if (name, seed) not in _models:
        _models[(name, seed)] = VononexModel(CONFIGS[name], seed=seed)
    return _models[(name, seed)]


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    err = float((got.double().cpu() - want).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err <= tol, err


# ---- each mechanism's kernel alone -----------------------------------------------------------------
@pytest.mark.parametrize("H, rows", [(72, None), (50, [3, 0, 3]), (4096, None)])
def test_rms_norm_of_a_scaled_sum(H, rows):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    x, d, w = torch.randn(5, H, generator=g), torch.randn(5, H, generator=g), torch.rand(H, generator=g) + 0.5
    want = VP.rms(1.7 * x.double() + d.double(), 1e-3, w.double() + 1.0)
    xs, out = x.to(DEV), torch.empty(5, H, device=DEV, dtype=torch.bfloat16)
    ops.rms_norm(xs, w.to(DEV), 1e-3, out_f32=xs, out_act=out, x_scale=1.7, delta=d.to(DEV), weight_offset=1.0)
    _close(xs, want, 1e-6)                                   # in place
    _close(out, want, 5e-3)
    if rows is not None:
        picked = torch.empty(len(rows), H, device=DEV)
        ops.rms_norm(x.to(DEV), None, 1e-3, out_f32=picked, rows=_i32(rows))
        _close(picked, VP.rms(x.double(), 1e-3)[rows], 1e-6)


def test_gated_activation_is_the_tanh_form():
    from transformers_neuronx_b200.kernels import ops
    gu = torch.randn(7, 2 * 50, generator=torch.Generator().manual_seed(2)) * 3
    out = torch.empty(7, 50, device=DEV)
    ops.gated_activation(gu.to(DEV), out, "gelu_pytorch_tanh")
    _close(out, VP.gelu_tanh(gu[:, :50].double()) * gu[:, 50:].double(), 1e-6)


@pytest.mark.parametrize("H, G, dk, dv, rot", [(6, 2, 24, 40, 16), (2, 1, 64, 64, 64), (3, 3, 10, 6, 0)])
def test_rotations_and_the_whole_projection_norm(H, G, dk, dv, rot):
    """q and k are normalised over all heads at once, then rotated on their first `rot` dims, q takes its head's
    number; values are rotated over all their dims; the output's turn back undoes the values' turn at equal positions."""
    from transformers_neuronx_b200.kernels import ops
    from transformers_neuronx_b200.parts.rotary import inverse_frequencies
    g = torch.Generator().manual_seed(3)
    N, D = 9, -(-max(dk, dv) // 16) * 16
    pos = [0, 1, 2, 15, 16, 17, 1000, 4095, 77]
    proj = torch.randn(N, 5 + H * dk + G * dk + G * dv, generator=g)
    wq, wk, temp = torch.rand(H * dk, generator=g) + 0.5, torch.rand(G * dk, generator=g) + 0.5, torch.rand(H, generator=g) + 0.5
    q, k, v = (torch.zeros(N, n * D, device=DEV) for n in (H, G, G))
    req = _i32([0] * (N - 1) + [-1])
    fq = inverse_frequencies(rot, 500.0, DEV) if rot else None
    fv = inverse_frequencies(dv, 500.0, DEV)
    ops.rotary_qkv_prep(proj.to(DEV), 5, 5 + H * dk, 5 + H * dk + G * dk, req, _i32(pos), wq.to(DEV), wk.to(DEV), 1e-4,
                        temp.to(DEV), fq, rot, fv, q, k, v, H, G, dk, dv, D)
    p = torch.tensor(pos)
    pq, pk, pv = proj[:, 5:5 + H * dk].double(), proj[:, 5 + H * dk:5 + H * dk + G * dk].double(), proj[:, 5 + H * dk + G * dk:].double()
    wantq = VP.turn(VP.rms(pq, 1e-4, wq.double()).view(N, H, dk), p, rot, 500.0) * temp.double()[None, :, None]
    wantk = VP.turn(VP.rms(pk, 1e-4, wk.double()).view(N, G, dk), p, rot, 500.0)
    wantv = VP.turn(pv.view(N, G, dv), p, dv, 500.0)
    for got, want, d in ((q, wantq, dk), (k, wantk, dk), (v, wantv, dv)):
        got = got.view(N, -1, D)
        _close(got[:6, :, :d], want[:6], 2e-6)                 # positions up to 17
        _close(got[6:-1, :, :d], want[6:-1], 3e-4)             # an angle of 4095 in 32-bit is exact to 2.4e-4
        assert float(got[:-1, :, d:].abs().max()) == 0.0 if D > d else True
    assert float(q[-1].abs().max()) == 0.0                     # the padded row is left alone
    out = torch.zeros(N, 3 + G * dv, device=DEV)
    ops.rotary_unrotate(v, req, _i32(pos), fv, 0.5, out[:, 3:], G, dv, D)
    _close(out[:-1, 3:], 0.5 * pv[:-1], 2e-4)                   # turned by p and back (32-bit angles of up to 4095)
    assert float(out[:, :3].abs().max()) == 0.0


@pytest.mark.parametrize("H, dk, dv", [(3, 20, 24), (2, 18, 10), (1, 128, 64), (2, 256, 16), (2, 8, 40)])
def test_retention_scan_carries_its_state_across_cuts_and_requests(H, dk, dv):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    T = 37
    q, k = torch.randn(2, T, H, dk, generator=g), torch.randn(2, T, H, dk, generator=g) * dk ** -0.5
    v = torch.randn(2, T, H, dv, generator=g)
    decay = torch.tensor([0.5, 0.99, 0.9999][:H])
    want = torch.zeros(2, T, H, dv, dtype=torch.float64)
    for r in range(2):
        for h in range(H):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            for t in range(T):
                S = float(decay[h]) * S + torch.outer(k[r, t, h].double(), v[r, t, h].double())
                want[r, t, h] = S.T @ q[r, t, h].double()
    state = torch.zeros(4, H, dv, dk, device=DEV)
    state[1].fill_(7.0)                                         # a slot nobody uses must stay as it is
    got = torch.zeros(2, T, H * dv)
    at = [0, 0]
    # request 0 in slot 2, request 1 in slot 0; portions of unequal sizes side by side, a padded request between
    for n0, n1 in [(5, 1), (1, 2), (8, 17), (1, 1), (22, 16)]:
        rows = torch.cat([q[0, at[0]:at[0] + n0], q[1, at[1]:at[1] + n1]]).reshape(n0 + n1, H * dk)
        krows = torch.cat([k[0, at[0]:at[0] + n0], k[1, at[1]:at[1] + n1]]).reshape(n0 + n1, H * dk)
        vrows = torch.cat([v[0, at[0]:at[0] + n0], v[1, at[1]:at[1] + n1]]).reshape(n0 + n1, H * dv)
        wide = torch.zeros(n0 + n1, 8 + H * dv)
        wide[:, 8:] = vrows
        out = torch.zeros(n0 + n1, H * dv, device=DEV)
        ops.retention_scan(rows.to(DEV), krows.to(DEV), wide.to(DEV)[:, 8:], decay.to(DEV), state,
                           _i32([0, 0, n0]), _i32([n0, 0, n1]), _i32([2, 1, 0]), out, H, dk, dv)
        got[0, at[0]:at[0] + n0], got[1, at[1]:at[1] + n1] = out[:n0].cpu(), out[n0:].cpu()
        at = [at[0] + n0, at[1] + n1]
    assert at == [T, T]
    _close(got.view(2, T, H, dv), want, 2e-5)
    assert float((state[1] - 7.0).abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0


@pytest.mark.parametrize("H, dk, dv, rot", [(3, 20, 24, 12), (2, 128, 64, 128), (1, 256, 16, 0), (2, 8, 40, 8)])
def test_retention_for_single_tokens_in_one_kernel(H, dk, dv, rot):
    """Rotation, state update, output, head-wise norm, gate and scale of a step of single tokens, against the
    equations: three requests (one of them padding) over four steps, from states that are not zero."""
    from transformers_neuronx_b200.kernels import ops
    from transformers_neuronx_b200.parts.rotary import inverse_frequencies
    g = torch.Generator().manual_seed(21)
    R, steps, pos0 = 2, 4, [37, 1000]
    wide = 3 + 2 * H * dk + 2 * H * dv
    proj = torch.randn(steps, R, wide, generator=g)
    decay = torch.tensor([0.5, 0.99, 0.9999][:H])
    state0 = torch.randn(4, H, dv, dk, generator=g) * 0.3
    slots = [2, 0]
    state = state0.clone().to(DEV)
    freq = inverse_frequencies(rot, 300.0, DEV) if rot else None
    want_state = state0.double().clone()
    for t in range(steps):
        out = torch.zeros(3, 5 + H * dv, device=DEV)
        rows = torch.zeros(3, wide)
        rows[0], rows[2] = proj[t, 0], proj[t, 1]                 # row 1 belongs to nobody
        ok = ops.retention_decode(rows.to(DEV), 3, 3 + H * dk, 3 + 2 * H * dk, 3 + 2 * H * dk + H * dv,
                                  _i32([pos0[0] + t, 0, pos0[1] + t]), freq, rot, dk ** -0.5, decay.to(DEV), state,
                                  _i32([0, 1, 2]), _i32([1, 0, 1]), _i32([slots[0], 3, slots[1]]), 1e-5, 0.8, out[:, 5:], H, dk, dv)
        assert ok
        for r in range(R):
            x = proj[t, r].double()
            p = torch.tensor([pos0[r] + t])
            q = VP.turn(x[3:3 + H * dk].view(1, H, dk), p, rot, 300.0)[0]
            k = VP.turn(x[3 + H * dk:3 + 2 * H * dk].view(1, H, dk), p, rot, 300.0)[0] * dk ** -0.5
            v = x[3 + 2 * H * dk:3 + 2 * H * dk + H * dv].view(H, dv)
            gate = x[3 + 2 * H * dk + H * dv:].view(H, dv)
            o = torch.zeros(H, dv, dtype=torch.float64)
            for h in range(H):
                S = float(decay[h]) * want_state[slots[r], h].T + torch.outer(k[h], v[h])      # stored [dv, dk]
                want_state[slots[r], h] = S.T
                o[h] = S.T @ q[h]
            want = 0.8 * VP.rms(o, 1e-5) * VP.silu(gate)
            _close(out[2 * r, 5:].view(H, dv), want, 3e-5 if pos0[r] < 100 else 3e-4)
        assert float(out[1].abs().max()) == 0.0 and float(out[:, :5].abs().max()) == 0.0
    _close(state, want_state, 3e-4)
    assert torch.equal(state[3].cpu(), state0[3]) and torch.equal(state[1].cpu(), state0[1])
    # sizes it does not take are refused without a launch, for the caller to run the three kernels
    assert ops.retention_decode(torch.zeros(1, 2 * 6 + 2 * 6, device=DEV), 0, 6, 12, 18, _i32([0]), None, 0, 1.0,
                                torch.ones(1, device=DEV), torch.zeros(1, 1, 6, 6, device=DEV), _i32([0]), _i32([1]), _i32([0]),
                                1e-5, 1.0, torch.zeros(1, 6, device=DEV), 1, 6, 6) is False


def test_headwise_norm_with_its_gate():
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    o, gate = torch.randn(6, 3 * 24, generator=g) * 50, torch.randn(6, 3 * 24, generator=g)
    out = torch.zeros(6, 4 + 72, device=DEV)
    ops.headwise_gated_rms_norm(o.to(DEV), gate.to(DEV), _i32([0] * 6), None, 1e-4, 1.3, out[:, 4:], 3, 24)
    want = 1.3 * VP.rms(o.double().view(6, 3, 24), 1e-4).reshape(6, 72) * VP.silu(gate.double())
    _close(out[:, 4:], want, 2e-6)


def test_mingru_scan_carries_its_state_across_cuts():
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    T, W = 200, 33
    proj = torch.randn(T, 3 * W + 2, generator=g) * 2
    z, u, gt = (proj[:, 2 + i * W:2 + (i + 1) * W].double() for i in range(3))
    zz, cand = torch.sigmoid(z), torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S, want = torch.zeros(W, dtype=torch.float64), []
    for t in range(T):
        S = (1 - zz[t]) * S + zz[t] * cand[t]
        want.append(S * VP.silu(gt[t]) * 0.7)
    state = torch.zeros(3, W, device=DEV)
    got, at = [], 0
    for n in (1, 2, 9, 1, 4, 24, 70, 89):           # the long portions are spread over several warps
        out = torch.zeros(n, W, device=DEV)
        ops.mingru_scan(proj[at:at + n].to(DEV), 2, 2 + W, 2 + 2 * W, state, _i32([0, 0]), _i32([0, n]), _i32([0, 2]),
                        out, W, out_scale=0.7)
        got.append(out.cpu()); at += n
    _close(torch.cat(got), torch.stack(want), 2e-6)
    _close(state[2], S, 2e-6)
    assert float(state[:2].abs().max()) == 0.0


# ---- whole models through the replay function ------------------------------------------------------
LENGTHS = {"P": [1, 2, 17, 45, 130], "Q": [3, 140, 300]}


def _requests(m, lengths, seed=100):
    return {f"r{i}": m.random_ids(n, seed=seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_whole_prompts(name, dtype):
    m = _model(name)
    reqs = _requests(m, LENGTHS[name])
    steps = whole_steps(reqs)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_a_prefix_then_token_by_token(name, dtype):
    """Decoding through the cache and the states: the last 40 tokens one by one (long enough for the decode
    steps to be replayed from a captured graph)."""
    m = _model(name)
    reqs = _requests(m, [n for n in LENGTHS[name] if n > 41])
    steps = cut_steps(reqs, [1000], tail=40)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype)


def test_from_the_first_token_on_one_by_one():
    m = _model("P")
    reqs = _requests(m, [50])
    steps = cut_steps(reqs, [1])
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_of_changing_size_down_to_two_tokens(name, dtype):
    m = _model(name)
    reqs = _requests(m, LENGTHS[name][-2:])
    steps = cut_steps(reqs, [2, 33, 3, 16, 2, 17, 64, 5, 130], tail=3)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype):
    """Eleven requests through four places: more requests than the replay program has slots, so a finished
    request's slot (its recurrent states) and its pages go to another request; the pool holds no more than the
    live requests need."""
    m = _model(name)
    lengths = [90, 7, 33, 150, 12, 64, 5, 49, 2, 120, 31] if name == "P" else [150, 20, 70, 9, 200, 40, 33, 129, 18]
    reqs = _requests(m, lengths, seed=300)
    steps = mixed_steps(reqs, [9, 2, 31, 16, 5, 64, 3])
    most = sorted(-(-n // 64) * 64 for n in lengths)[-4:]
    res = run_trace_inprocess(m.folder, dtype, steps, sum(most))
    compare(m, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_no_fast_path_takes(dtype):
    m = _model("R")
    reqs = _requests(m, [3, 70, 41], seed=600)
    for steps in (whole_steps(reqs), mixed_steps(reqs, [7, 2, 19, 33], decode_tail=12)):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 4), dtype)


def test_logits_do_not_depend_on_the_cut_or_the_batch_beyond_rounding():
    m = _model("P")
    reqs = _requests(m, [130, 45], seed=500)
    runs = []
    for steps in (whole_steps(reqs), cut_steps(reqs, [2, 16, 17, 1, 31]), mixed_steps(reqs, [15, 2, 40], decode_tail=20)):
        res = run_trace_inprocess(m.folder, "float32", steps, 64 * 4)
        at, out = {r: 0 for r in reqs}, {}
        for s in steps:
            row = 0
            for e in s["entries"]:
                for w in e["want"]:
                    out[(e["id"], at[e["id"]] + w)] = torch.from_numpy(res[s["step"]][row].copy()); row += 1
                at[e["id"]] += len(e["tokens"])
        runs.append(out)
    for other in runs[1:]:
        for key, lg in other.items():
            assert float((lg - runs[0][key]).abs().max()) <= 2e-5 * float(runs[0][key].abs().max()), key


# ---- far keys, made to stand out -------------------------------------------------------------------
def _one_layer(left_scale, right_scale, decay):
    return {"architecture": "Vononex", "vocab": 97, "width": 64, "postln_alpha": 1.0, "norm": {"eps": 1e-5},
            "init_std": 0.3, "layers": [parallel(left(4, 2, 32, 16, 0.25, 32, 10000.0), right(2, 16, 32, decay, 16, 100.0),
                                                 left_scale, right_scale, None)]}


def test_a_sharp_softmax_finds_the_same_far_key():
    """Head temperatures of 40 make every head's softmax nearly one-hot over 300 keys: a key that is off by one
    position, a page that is mixed up or a rotation that is wrong picks another value and changes the logits
    wholesale.  Retention is switched off by its scale."""
    def sharp(t):
        t["l0.mix.left.temp"] = torch.full_like(t["l0.mix.left.temp"], 40.0)
    m = VononexModel(_one_layer(1.0, 0.0, [0.9, 0.9]), seed=8, edit=sharp)
    reqs = {"a": m.random_ids(300, 1), "b": m.random_ids(77, 2)}
    plain = m.plain_logits(reqs["a"])
    for steps in (whole_steps(reqs), cut_steps(reqs, [16, 15, 2, 33, 1, 64], tail=20), mixed_steps(reqs, [31, 2, 17])):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 7), "float32", tol=2e-4)
    assert float(plain.std()) > 0.05


def test_a_slow_decay_remembers_the_first_tokens():
    """Decays of 0.99999 and 1 - 2^-12 keep the first token's outer product in the state for the whole prompt;
    attention is switched off by its scale."""
    m = VononexModel(_one_layer(0.0, 1.0, [0.99999, 1 - 2.0 ** -12]), seed=9)
    reqs = {"a": m.random_ids(260, 3)}
    for steps in (whole_steps(reqs), cut_steps(reqs, [2, 50, 1, 17], tail=30)):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 5), "float32")


def test_long_decoding():
    m = _model("P")
    reqs = _requests(m, [260], seed=700)
    steps = cut_steps(reqs, [4], tail=250)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 5), "float32")


# ---- the engine's own entry point ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype):
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    m = _model("Q")
    model, typed = load_model(m.folder, dtype, verbose=False)
    eng = LLMEngine(model, EngineConfig(dtype=dtype, max_num_seqs=3, max_batch_tokens=48, max_portion=20, max_tokens=640,
                                        max_model_len=256))
    prompts = [m.random_ids(n, 900 + n) for n in (37, 5, 70, 18)]
    outs = eng.generate(prompts, 12, stop_on_eos=False)
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        logits = m.plain_logits(list(prompt) + list(out))
        for i, tok in enumerate(out):
            lg = logits[len(prompt) - 1 + i]
            if tok != int(lg.argmax()):                      # a tie that rounding may decide either way
                assert float(lg.max() - lg[tok]) / float(lg.abs().max()) <= 2 * TOLERANCE[dtype], (i, tok)
    eng.runner.cache.check()
    assert eng.runner.cache.slots.num_free == 3


def test_the_entry_point_class_and_the_command_line(tmp_path):
    """config.json picks the entry-point class; greedy `sample` equals the plain argmax, teacher-forced; the demo
    command line writes a folder of random weights from a config.json and samples from it."""
    import json
    import os
    import subprocess
    import sys
    from transformers_neuronx_b200 import NeuronAutoModelForCausalLM, VononexForSampling
    m = _model("P")
    model = NeuronAutoModelForCausalLM.from_pretrained(m.folder, batch_size=2, amp="f32", n_positions=64)
    assert isinstance(model, VononexForSampling)
    model.to_neuron()
    prompts = torch.tensor([m.random_ids(9, 41), m.random_ids(9, 42)])
    seq = model.sample(prompts, sequence_length=20, top_k=1)
    assert tuple(seq.shape) == (2, 20) and torch.equal(seq[:, :9], prompts)
    for row in seq.tolist():
        logits = m.plain_logits(row)
        for i in range(9, 20):
            lg = logits[i - 1]
            if row[i] != int(lg.argmax()):
                assert float(lg.max() - lg[row[i]]) / float(lg.abs().max()) <= 1e-4
                break
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    demo = os.path.join(root, "bin", "vononex_demo")
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(CONFIG_P))
    folder = tmp_path / "model"
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "save", str(folder), "--random", "--config", str(cfg)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "run", str(folder), "--batch_size", "2", "--n_positions", "24",
                        "--top_k", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "generated_sequence=" in r.stdout, r.stderr
