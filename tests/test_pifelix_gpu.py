"""The Pifelix decoder on the GPU against the plain implementation (tests/plain/pifelix_plain.py): every mechanism's
kernel alone, then whole models through the replay program's function (whole prompts, token by token, portions down
to two tokens, mixed batches with pages and slots used again), keys at the edges of chunks made to stand out, long
decoding, and greedy generation through the engine's own entry point and scheduler."""
import copy
import math
from types import SimpleNamespace

import pytest
import torch

from helpers import run_trace_inprocess
from pifelix_helpers import (CONFIG_A, CONFIGS, PifelixModel, attention, compare, compare_rows, cut_steps, experts, layer,
                             mixed_steps, rot, whole_steps)
from plain import pifelix_plain as PP
from vononex_helpers import TOLERANCE

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
_models = {}


def _model(name, seed=5):
    if (name, seed) not in _models:
        _models[(name, seed)] = PifelixModel(CONFIGS[name], seed=seed)
    return _models[(name, seed)]


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _close(got, want, tol):
    err = float((got.double().cpu() - want.double()).abs().max()) / max(float(want.abs().max()), 1e-30)
    assert err <= tol, err


# ---- each mechanism's kernel alone -----------------------------------------------------------------
@pytest.mark.parametrize("H", [72, 50, 4096])
def test_the_norm_of_a_sublayers_output_is_added_to_the_stream(H):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    x, d, w = torch.randn(5, H, generator=g), torch.randn(5, H, generator=g) * 30, torch.rand(H, generator=g) + 0.5
    want = x.double() + 0.3 * PP.rms(d.double(), 1e-3, w.double())
    xs, out = x.to(DEV), torch.empty(5, H, device=DEV, dtype=torch.bfloat16)
    ops.rms_norm_add(xs, 0.3, d.to(DEV), w.to(DEV), 1e-3, out_f32=xs, out_act=out)
    _close(xs, want, 1e-6)                                   # in place
    _close(out, want, 5e-3)


def test_the_embedding_is_scaled_in_32_bit():
    from transformers_neuronx_b200.kernels import ops
    table = torch.randn(9, 40, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    x, xa = torch.empty(4, 40, device=DEV), torch.empty(4, 40, device=DEV, dtype=torch.bfloat16)
    ops.embed(table.to(DEV), None, _i32([3, 0, 8, 3]), None, _i32([0, 1, 2, 3]), 0, x, xa, tok_scale=17.25)
    want = table[[3, 0, 8, 3]].double() * 17.25
    _close(x, want, 1e-7)
    _close(xa, want, 4e-3)


def _step_arrays(cuts):
    """cuts: per request (slot, first position, rows) -> the index arrays of a step, as the step function packs them."""
    req, pos, q_start, q_len, slots, row = [], [], [], [], [], 0
    for r, (slot, first, n) in enumerate(cuts):
        req += [r] * n
        pos += list(range(first, first + n))
        q_start.append(row); q_len.append(n); slots.append(slot)
        row += n
    return req, pos, q_start, q_len, slots


@pytest.mark.parametrize("H, G, dk, dv, taps, rdims, inter, scaling, dtype", [
    (6, 2, 24, 40, 4, 16, True, (2.5, 64, 16.0, 2.0), torch.float32),
    (2, 1, 64, 64, 2, 64, True, None, torch.float32),
    (3, 3, 10, 6, 3, 0, True, None, torch.float32),
    (4, 0, 32, 32, 3, 32, True, (4.0, 32, 8.0, 1.0), torch.float32),       # queries only: a layer that reads another's pages
    (2, 2, 128, 96, 8, 64, False, None, torch.float32),                   # pairs (i, i + dims/2) as other designs want them
    (5, 1, 48, 48, 1, 48, True, None, torch.float32),                     # one tap: a scale per channel, nothing kept
    (4, 2, 64, 48, 3, 64, True, (4.0, 512, 32.0, 1.0), torch.bfloat16),
    (3, 1, 96, 32, 4, 40, True, None, torch.bfloat16),                    # 12 lanes a head, two heads a warp, a padded value head
    (2, 2, 256, 8, 2, 256, True, None, torch.float32),
])
@pytest.mark.parametrize("col0", [5, 8])                                  # 8: the addresses allow the kernel of 8-channel pieces
def test_convolution_norm_and_rotation_across_cuts(H, G, dk, dv, taps, rdims, inter, scaling, dtype, col0):
    """Two requests cut into unequal steps side by side (single tokens, pairs, a padded row, a request left out of a
    step): what a token reads from the state equals what it would have read from the rows of a longer step."""
    from transformers_neuronx_b200.kernels import ops
    from transformers_neuronx_b200.parts.rotary import inverse_frequencies, rotation_magnitude
    from transformers_neuronx_b200.parts.spec import FrequencyRampSpec
    g = torch.Generator().manual_seed(3)
    T, D, C = 41, -(-max(dk, dv) // 16) * 16, H * dk + G * (dk + dv)
    u = (torch.randn(2, T, C, generator=g)).to(dtype)
    w = torch.randn(C, taps, generator=g)
    gq, gk = torch.rand(dk, generator=g) + 0.5, torch.rand(dk, generator=g) + 0.5
    rspec = {"dims": rdims, "base": 500.0}
    if scaling:
        rspec["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    fs = FrequencyRampSpec(*scaling) if scaling else None
    freq = inverse_frequencies(rdims, 500.0, DEV, fs) if rdims else None
    want = []
    for r in range(2):
        y = PP.short_conv(u[r].double(), w.double())
        q = PP.rms(y[:, :H * dk].view(T, H, dk), 1e-4, gq.double())
        k = PP.rms(y[:, H * dk:H * dk + G * dk].view(T, G, dk), 1e-4, gk.double()) if G else None
        if inter:
            q, k = PP.turn_pairs(q, range(T), rspec), (PP.turn_pairs(k, range(T), rspec) if G else None)
        elif rdims:                                            # halves: the same turn on a permuted head
            perm = [i // 2 + (rdims // 2) * (i % 2) for i in range(rdims)] + list(range(rdims, dk))
            inv = [perm.index(i) for i in range(dk)]
            q, k = PP.turn_pairs(q[..., perm], range(T), rspec)[..., inv], PP.turn_pairs(k[..., perm], range(T), rspec)[..., inv]
        want.append((q, k, y[:, H * dk + G * dk:].view(T, G, dv) if G else None))
    keep = taps - 1
    state = torch.zeros(4, keep, C, device=DEV, dtype=dtype) if keep else None
    if keep:
        state[1].fill_(7.0)                                     # a slot nobody uses must stay as it is
    got = [[torch.zeros(T, n, D) for n in (H, G, G)] for _ in range(2)]
    at = [0, 0]
    for n0, n1 in [(5, 1), (1, 2), (2, 0), (1, 1), (8, 17), (1, 1), (23, 19)]:
        cuts = [(slot, at[r], n) for r, (slot, n) in enumerate(((2, n0), (0, n1))) if n]
        reqs = [r for r, n in enumerate((n0, n1)) if n]
        req, pos, q_start, q_len, slots = _step_arrays(cuts)
        rows = torch.cat([u[r, at[r]:at[r] + n] for r, n in zip(reqs, [c[2] for c in cuts])])
        N = rows.shape[0]
        proj = torch.zeros(N + 1, (col0 + C + 3) if col0 % 8 else -(-(col0 + C + 3) // 8) * 8, dtype=dtype)
        proj[:N, col0:col0 + C] = rows
        ctx = SimpleNamespace(token_request=_i32(req + [-1]), positions=_i32(pos + [0]), q_start=_i32(q_start + [0]),
                              q_len=_i32(q_len + [0]), state_slots=_i32(slots + [-1]), decode_only=all(n == 1 for n in q_len))
        qo, ko, vo = (torch.full((N + 1, n * D), 9.0, device=DEV, dtype=dtype) for n in (H, max(G, 1), max(G, 1)))
        ops.conv_qkv_prep(proj.to(DEV), col0, w.t().contiguous().to(DEV), taps, state, ctx, gq.to(DEV), gk.to(DEV) if G else None, 1e-4, freq,
                          rdims, inter, rotation_magnitude(fs), qo, ko if G else None, vo if G else None, H, G, dk, dv, D)
        assert float((qo[N].float() - 9.0).abs().max()) == 0.0   # the padded row is left alone
        row = 0
        for r, (_, first, n) in zip(reqs, cuts):
            for j, o in enumerate((qo, ko, vo)[:3 if G else 1]):
                got[r][j][first:first + n] = o[row:row + n].float().cpu().view(n, -1, D)
            row += n; at[r] += n
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    for r in range(2):
        for j, d in ((0, dk), (1, dk), (2, dv)):
            if want[r][j] is None:
                continue
            _close(got[r][j][..., :d], want[r][j], tol)
            assert D == d or float(got[r][j][..., d:].abs().max()) == 0.0
    if keep:
        assert float((state[1].float() - 7.0).abs().max()) == 0.0
        _close(state[2].float(), u[0, T - keep:].double(), 0.0)   # the request's last projected values, oldest first
        _close(state[0].float(), u[1, T - keep:].double(), 0.0)


@pytest.mark.parametrize("chunk", [1, 16, 20, 33, 64, 96, 500])
@pytest.mark.parametrize("n_heads, n_kv, d", [(4, 2, 64), (6, 2, 48), (2, 2, 128)])
def test_the_chunked_mask_in_every_attention_kernel(chunk, n_heads, n_kv, d):
    """Contexts and portions that begin and end just before, at and just after the edges of chunks; one far key
    planted per request (tests/test_kernels_gpu.py: PagedCase) that a query sees only if it lies in its chunk."""
    from test_kernels_gpu import PagedCase, rel_err
    from transformers_neuronx_b200.kernels import ops as o
    c = chunk
    lens = [(0, 2), (0, 130), (c - 1 if c > 1 else 3, 1), (c, 1), (2 * c + 1, 1), (3 * c - 1, 70), (c // 2, c + 3), (199, 1),
            (64, 129), (5 * c, 2), (333, 1)]
    scale = 1.0 / math.sqrt(d)
    for kind, dtype in (("prefill_tc", torch.bfloat16), ("prefill", torch.bfloat16), ("decode", torch.bfloat16),
                        ("simt", torch.bfloat16), ("simt", torch.float32)):
        if kind == "prefill_tc" and d not in (64, 80, 96, 112, 128):
            continue
        case = PagedCase(lens, n_heads, n_kv, d, dtype, seed=31 + d + chunk, **({"poison": 3.0e4} if kind == "prefill_tc" else {}))
        want = torch.cat([PP.chunked_attention(q.double(), k.double(), v.double(), scale, chunk, first_query=cl).reshape(ql, -1)
                          for (cl, ql), q, k, v in zip(case.lens, case.q, case.k, case.v)]).to(DEV)
        out = torch.zeros(case.N, n_heads * d, dtype=dtype, device=DEV)
        multi = torch.ones(case.N, dtype=torch.bool, device=DEV)
        multi[case.decode_rows.long()] = False
        args = (case.q_flat, case.cache, case.bt, case.tile_req, case.tile_q0, case.q_start, case.q_len, case.ctx_len, out,
                n_heads, scale)
        if kind == "prefill_tc":
            o.attention_prefill_tc(*args, chunk=chunk); rows = multi
        elif kind == "prefill":
            o.attention_prefill(*args, chunk=chunk); rows = multi
        elif kind == "decode":
            o.attention_decode(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, n_heads, scale,
                               rows=case.decode_rows, max_kv_len=5 * c + 400, chunk=chunk)
            rows = ~multi
        else:
            o.attention_simt(case.q_flat, case.cache, case.bt, case.tok_req, case.positions, out, n_heads, scale, chunk=chunk)
            rows = torch.ones_like(multi)
        o.raise_on_device_error()
        assert torch.isfinite(out.float()).all(), kind
        assert rel_err(out[rows], want[rows]) <= (1.5e-2 if dtype != torch.float32 else 1e-5), kind
    with pytest.raises(o.KernelError, match="not both"):
        o.mask_rule(window=5, chunk=4)


@pytest.mark.parametrize("W, E, top, F, dtype, softmax, renorm, on_input", [
    (72, 5, 2, 36, torch.float32, False, False, True),
    (100, 7, 7, 30, torch.float32, False, False, True),
    (256, 8, 1, 128, torch.bfloat16, False, False, True),
    (64, 40, 8, 24, torch.float32, True, True, False),        # what other designs do: softmax, renormalised, on the output
    (48, 20, 16, 16, torch.float32, False, False, True),
    (320, 3, 2, 50, torch.bfloat16, False, False, True),
])
def test_routing_and_experts(W, E, top, F, dtype, softmax, renorm, on_input):
    from transformers_neuronx_b200.kernels import ops
    g = torch.Generator().manual_seed(7)
    N = 37
    h = torch.randn(N, W, generator=g).to(dtype)
    router = (torch.randn(E, W, generator=g) * 0.3).to(torch.bfloat16)
    gate_up = (torch.randn(E, 2 * F, W, generator=g) * W ** -0.5 * 3).to(torch.bfloat16)
    down = (torch.randn(E, W, F, generator=g) * F ** -0.5).to(torch.bfloat16)
    req = [0] * (N - 1) + [-1]
    ids = torch.full((N, top), -7, dtype=torch.int32, device=DEV)
    wts = torch.zeros(N, top, device=DEV)
    ops.moe_route(h.to(DEV), router.to(DEV), _i32(req), ids, wts, top, softmax_scores=softmax, renormalize=renorm)
    z = h.double() @ router.double().T
    score = torch.softmax(z, -1) if softmax else torch.sigmoid(z)
    lim, out_want = 1.5, torch.zeros(N, W, dtype=torch.float64)
    for n in range(N - 1):
        order = sorted(range(E), key=lambda e: (-float(score[n, e]), e))[:top]
        got = ids[n].tolist()
        if got != order:                                       # two scores that rounding may order either way
            assert sorted(got) == sorted(order) or min(abs(float(score[n, a] - score[n, b])) for a in got for b in order if a != b) < 1e-3
        ws = score[n, got] / (score[n, got].sum() if renorm else 1.0)
        _close(wts[n], ws, 2e-6 if dtype == torch.float32 else 1e-2)
        for e, wgt in zip(got, ws):
            x = h[n].double() * (float(wgt) if on_input else 1.0)
            gt = torch.clamp(gate_up[e, :F].double() @ x, max=lim)
            up = torch.clamp(gate_up[e, F:].double() @ x, -lim, lim)
            out_want[n] += (1.0 if on_input else float(wgt)) * (down[e].double() @ (gt * torch.sigmoid(1.702 * gt) * (up + 1.0)))
    assert ids[N - 1].tolist() == [-1] * top                   # the padded row chooses nobody
    y = torch.empty(N * top, F, device=DEV, dtype=dtype)
    out = torch.full((N, W), 2.0, device=DEV)
    ops.moe_experts(h.to(DEV), gate_up.to(DEV), down.to(DEV), ids, wts, y, out, lim, -lim, lim, 1.702, 1.0,
                    weight_on_input=on_input, accumulate=True)
    _close(out[:N - 1] - 2.0, out_want[:N - 1], 3e-6 if dtype == torch.float32 else 2e-2)
    assert float((out[N - 1] - 2.0).abs().max()) == 0.0
    ops.moe_experts(h.to(DEV), gate_up.to(DEV), down.to(DEV), ids, wts, y, out, lim, -lim, lim, 1.702, 1.0,
                    weight_on_input=on_input, accumulate=False)
    _close(out[:N - 1], out_want[:N - 1], 3e-6 if dtype == torch.float32 else 2e-2)


# ---- whole models through the replay program's function ----------------------------------------------
LENGTHS = {"A": [1, 2, 19, 20, 21, 70, 133], "B": [3, 64, 65, 200, 150]}


def _requests(m, lengths, seed=100):
    return {f"r{i}": m.random_ids(n, seed=seed + i) for i, n in enumerate(lengths)}


def test_the_residual_stream_after_every_layer():
    from transformers_neuronx_b200.engine.loading import load_model
    from transformers_neuronx_b200.engine.step import StepEntry, StepRunner
    m = _model("A")
    ids = m.random_ids(47, 11)
    model, _ = load_model(m.folder, "float32", verbose=False)
    runner = StepRunner(model, page_size=16, num_pages=8, max_slots=2, max_model_len=256)
    runner.add_request("a")
    with model.tap_hidden_states() as taps:
        runner.step([StepEntry("a", ids, [46])])
        want = m.plain_hidden(ids)
        for i in range(len(CONFIG_A["layers"])):
            _close(taps[f"entry{i}"], want[i], 2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts(name, dtype):
    m = _model(name)
    reqs = _requests(m, LENGTHS[name])
    steps = whole_steps(reqs)
    compare_rows(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_prefix_then_token_by_token(name, dtype):
    """Decoding through the pages and the convolutions' states: the last 70 tokens one by one, across several edges of
    chunks (long enough for the decode steps to be replayed from a captured graph)."""
    m = _model(name)
    reqs = _requests(m, [n for n in LENGTHS[name] if n > 71])
    steps = cut_steps(reqs, [1000], tail=70)
    compare_rows(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype)


@pytest.mark.parametrize("name", ["A", "C"])
def test_from_the_first_token_on_one_by_one(name):
    m = _model(name)
    reqs = _requests(m, [50])
    steps = cut_steps(reqs, [1])
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_of_changing_size_down_to_two_tokens(name, dtype):
    m = _model(name)
    reqs = _requests(m, LENGTHS[name][-2:])
    steps = cut_steps(reqs, [2, 33, 3, 16, 2, 17, 64, 5, 130], tail=3)
    compare_rows(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 5), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype):
    """Eleven requests through four places: more requests than the replay program has slots, so a finished request's
    slot (the pasts of its convolutions) and its pages go to another request; the pool holds no more than the live
    requests need, and pages before the running chunk have gone back to it meanwhile."""
    m = _model(name)
    lengths = [90, 7, 33, 150, 12, 64, 5, 49, 2, 120, 31] if name == "A" else [150, 20, 70, 9, 200, 40, 33, 129, 18]
    reqs = _requests(m, lengths, seed=300)
    steps = mixed_steps(reqs, [9, 2, 31, 16, 5, 64, 3])
    most = sorted(-(-n // 64) * 64 for n in lengths)[-4:]
    res = run_trace_inprocess(m.folder, dtype, steps, sum(most))
    compare_rows(m, reqs, steps, res, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_no_fast_path_takes(dtype):
    m = _model("C")
    reqs = _requests(m, [3, 70, 41], seed=600)
    for steps in (whole_steps(reqs), mixed_steps(reqs, [7, 2, 19, 33], decode_tail=12)):
        compare_rows(m, reqs, steps, run_trace_inprocess(m.folder, dtype, steps, 64 * 4), dtype)


def test_logits_do_not_depend_on_the_cut_or_the_batch_beyond_rounding():
    m = _model("A")
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


# ---- keys at the edges of chunks, made to stand out --------------------------------------------------
def _one_layer(chunk, scale, taps=3, kv_from_too=False, top=2):
    att = attention(4, 2, 32, 16, scale, taps, chunk, rot(32, 10000.0, (3.0, 48, 12.0, 1.5)))
    layers = [layer(att, None)]
    if kv_from_too:
        layers.append(layer(dict(copy.deepcopy(att), kv_from=0), experts(4, top, 32, 3.0)))
    return {"architecture": "Pifelix", "vocab": 97, "width": 64, "residual_mult": 1.0, "embedding": {"scale": 8.0},
            "norm": {"eps": 1e-5}, "init_std": 0.3, "layers": layers}


@pytest.mark.parametrize("chunk", [16, 23, 64])
def test_a_sharp_softmax_finds_the_same_key_at_the_edges_of_chunks(chunk):
    """A scale of 40 on unit-norm queries and keys makes every head's softmax nearly one-hot: a mask that is one
    position off, a page that is mixed up or a rotation that is wrong picks another key's value wherever the best
    key sits at the chunk's first position or just before it, and changes the logits wholesale.  The second layer
    reads the first one's pages."""
    def unit(t):
        for k in list(t):
            if k.endswith(".norm") and ".mix." in k:
                t[k] = torch.ones_like(t[k])
    m = PifelixModel(_one_layer(chunk, 40.0 / 32 ** 0.5, kv_from_too=True), seed=8, edit=unit)
    reqs = {"a": m.random_ids(300, 1), "b": m.random_ids(77, 2)}
    plain = m.plain_logits(reqs["a"])
    for steps in (whole_steps(reqs), cut_steps(reqs, [16, 15, 2, 33, 1, 64], tail=2 * chunk + 3), mixed_steps(reqs, [31, 2, 17])):
        compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 7), "float32", tol=2e-4)
    assert float(plain.std()) > 0.05


def test_the_first_tokens_see_zeros_before_the_sequence():
    """Eight taps: the first seven positions of every request read zeros for what lies before position 0, whatever
    the slot held before (the second request takes the first one's slot)."""
    m = PifelixModel(_one_layer(40, 0.2, taps=8), seed=9)
    reqs = {"a": m.random_ids(30, 3), "b": m.random_ids(9, 4), "c": m.random_ids(12, 5)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"], "want": list(range(30))}], "end": ["a"]}]
    steps += [{"step": 1 + i, "entries": [{"id": "b", "tokens": [t], "want": [0]}], "end": ["b"] if i == 8 else []}
              for i, t in enumerate(reqs["b"])]
    steps += [{"step": 10, "entries": [{"id": "c", "tokens": reqs["c"][:2], "want": [0, 1]}], "end": []},
              {"step": 11, "entries": [{"id": "c", "tokens": reqs["c"][2:5], "want": [0, 1, 2]}], "end": []},
              {"step": 12, "entries": [{"id": "c", "tokens": reqs["c"][5:], "want": list(range(7))}], "end": ["c"]}]
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64), "float32")


def test_long_decoding():
    m = _model("A")
    reqs = _requests(m, [260], seed=700)
    steps = cut_steps(reqs, [4], tail=250)
    compare(m, reqs, steps, run_trace_inprocess(m.folder, "float32", steps, 64 * 5), "float32")


# ---- the engine's own entry point ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype):
    from transformers_neuronx_b200.config import EngineConfig
    from transformers_neuronx_b200.engine import LLMEngine, load_model
    m = _model("B")
    model, typed = load_model(m.folder, dtype, verbose=False)
    eng = LLMEngine(model, EngineConfig(dtype=dtype, max_num_seqs=3, max_batch_tokens=48, max_portion=20, max_tokens=640,
                                        max_model_len=256))
    prompts = [m.random_ids(n, 900 + n) for n in (37, 5, 70, 18)]
    outs = eng.generate(prompts, 12, stop_on_eos=False)
    off = 0
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        logits = m.plain_logits(list(prompt) + list(out))
        for i, tok in enumerate(out):
            lg = logits[len(prompt) - 1 + i]
            if tok != int(lg.argmax()):                      # a tie that rounding may decide either way
                off += float(lg.max() - lg[tok]) / float(lg.abs().max()) > 2 * TOLERANCE[dtype]
    # in bfloat16 a token between two experts may take the other one; in 32-bit every token is the plain argmax or its tie
    assert off <= (0 if dtype == "float32" else 3), off
    eng.runner.cache.check()
    assert eng.runner.cache.slots.num_free == 3


def test_the_entry_point_class_and_the_command_line(tmp_path):
    """config.json picks the entry-point class; greedy `sample` equals the plain argmax, teacher-forced; the demo
    command line writes a folder of random weights from a config.json and samples from it."""
    import json
    import os
    import subprocess
    import sys
    from transformers_neuronx_b200 import NeuronAutoModelForCausalLM, PifelixForSampling
    m = _model("A")
    model = NeuronAutoModelForCausalLM.from_pretrained(m.folder, batch_size=2, amp="f32", n_positions=64)
    assert isinstance(model, PifelixForSampling)
    model.to_neuron()
    prompts = torch.tensor([m.random_ids(9, 41), m.random_ids(9, 42)])
    seq = model.sample(prompts, sequence_length=30, top_k=1)
    assert tuple(seq.shape) == (2, 30) and torch.equal(seq[:, :9], prompts)
    for row in seq.tolist():
        logits = m.plain_logits(row)
        for i in range(9, 30):
            lg = logits[i - 1]
            if row[i] != int(lg.argmax()):
                assert float(lg.max() - lg[row[i]]) / float(lg.abs().max()) <= 1e-4
                break
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    demo = os.path.join(root, "bin", "pifelix_demo")
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(CONFIG_A))
    folder = tmp_path / "model"
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "save", str(folder), "--random", "--config", str(cfg)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([sys.executable, demo, "--amp", "bf16", "run", str(folder), "--batch_size", "2", "--n_positions", "24",
                        "--top_k", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "generated_sequence=" in r.stdout, r.stderr


@pytest.mark.parametrize("N, W, E, top, F, on_input", [(300, 256, 8, 2, 128, True), (129, 320, 3, 3, 72, True),
                                                      (1000, 64, 40, 1, 200, False), (64, 128, 5, 4, 64, True),
                                                      (2, 2048, 8, 2, 2816, True), (9, 256, 8, 2, 136, True),      # tiles of 16
                                                      (40, 512, 4, 1, 264, True), (70, 384, 6, 2, 1000, False)])   # of 32 and 64
def test_experts_as_grouped_products_equal_the_streamed_form(N, W, E, top, F, on_input):
    """Many rows: the pairs sorted by expert into tiles of 128 rows and run on the tensor cores, against the form that
    streams an expert's matrices per row (which test_routing_and_experts holds against the plain implementation), with a
    padded row, experts nobody chooses and an expert that takes more than one tile."""
    from transformers_neuronx_b200.kernels import ops
    from transformers_neuronx_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(11)
    h = torch.randn(N, W, generator=g).to(torch.bfloat16).to(DEV)
    router = (torch.randn(E, W, generator=g) * 0.3)
    router[0] += 0.4 * router[1]                                   # lopsided: some experts get most of the rows
    gate_up = (torch.randn(E, 2 * F, W, generator=g) * W ** -0.5 * 3).to(torch.bfloat16).to(DEV)
    down = (torch.randn(E, W, F, generator=g) * F ** -0.5).to(torch.bfloat16).to(DEV)
    req = _i32([0] * (N - 1) + [-1])
    ids, wts = torch.empty(N, top, dtype=torch.int32, device=DEV), torch.empty(N, top, device=DEV)
    ops.moe_route(h, router.to(torch.bfloat16).to(DEV), req, ids, wts, top)
    assert ops.moe_grouped_supported(h, gate_up, down)
    y = torch.empty(N * top, F, device=DEV, dtype=torch.bfloat16)
    want, got = torch.full((N, W), 1.5, device=DEV), torch.full((N, W), 1.5, device=DEV)
    for acc in (True, False):
        ops.moe_experts(h, gate_up, down, ids, wts, y, want, 1.5, -1.5, 1.5, 1.702, 1.0, weight_on_input=on_input, accumulate=acc)
        ctx = StepContext(torch.device(DEV), torch.bfloat16)
        ops.moe_grouped(ctx, h, gate_up, down, ids, wts, got, 1.5, -1.5, 1.5, 1.702, 1.0, weight_on_input=on_input, accumulate=acc)
        ops.raise_on_device_error()
        assert torch.isfinite(got).all()
        # both round g, u and y to bfloat16 at the same places; the sums run in another order
        assert float((got - want).abs().max()) <= 2e-2 * float(want.abs().max())
        assert float((got[N - 1] - 1.5).abs().max()) == 0.0        # the padded row is left alone
