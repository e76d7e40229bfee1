"""The Fudulix design on the CPU: its configuration reader, the plain statement's own
mechanisms on values computed by hand, and the engine's host logic (the previous token and
the convolutions' inputs in state slots, pages kept for the first tokens of a windowed
layer, values handed from layer to layer inside a step, batching) with the kernels
replaced by their plain statements (tests/host_ops.py)."""
import copy
import math

import pytest
import torch

import fudulix_cases as fk
import host_ops
import model_cases as mc
import plain_fudulix as plain
import traces
from inferx_b200.cache.manager import CacheGroup, CacheManager
from inferx_b200.config.model_config import ConfigError
from inferx_b200.config.registry import config_from_json
from inferx_b200.engine.replay import ReplaySession

CASES = [("FA", fk.FA, 0, [5, 9, 17, 40, 3, 70], 4), ("FB", fk.FB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("FC", fk.FC, 3, [21, 1, 50, 2, 37], 16)]
D = torch.float64


# -- configuration ---------------------------------------------------------------
def test_config_reads_every_size_and_constant():
    cfg, spec = config_from_json(fk.FA)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.buckets, cfg.mul_prev, cfg.mul_cur) == \
        (211, 96, 1e-6, 53, 5, 3)
    e = spec.embedding
    assert (e.kind, e.buckets, e.mul_prev, e.mul_cur, e.norm.eps) == \
        ("pair_embedding", 53, 5, 3, 1e-6)
    a, b, c, d = (l.mixer for l in spec.layers)
    assert (a.heads, a.kv_heads, a.head_dim, a.value_dim, a.scale, a.window, a.keep_first,
            a.conv_taps) == (4, 2, 24, 16, 0.3, 9, 3, 3)
    assert a.projection_norm and not a.head_unit_norm and not a.sink
    assert (a.position.layout, a.position.rotary_dim, a.position.theta, a.position.scaling) == \
        ("half", 12, 5000.0, ("ramp", 3.0, 64.0, 8.0, 1.0))
    assert (b.heads, b.kv_heads, b.head_dim, b.value_dim, b.window, b.keep_first,
            b.conv_taps) == (6, 2, 16, 16, 7, 0, 0)
    assert b.head_unit_norm and b.sink and not b.projection_norm
    assert (b.position.layout, b.position.scaling) == \
        ("interleaved", ("wavelength", 4.0, 1.0, 4.0, 32.0))
    # the first layer that mixes leaves its values, later ones blend, the last does neither
    assert [m.value_mix for m in (a, b, c, d)] == ["source", "mix", "mix", "none"]
    assert d.position is None and d.conv_taps == 0
    f0, f1, f2 = (spec.layers[i].ffn for i in range(3))
    assert (f0.kind, f0.intermediate, f0.activation, f0.bias) == ("glu_biased", 72, "gelu_tanh",
                                                                  True)
    assert (f1.num_experts, f1.identity_experts, f1.top_k, f1.group_count, f1.group_keep,
            f1.expert_intermediate, f1.shared.intermediate, f1.renorm_eps) == \
        (5, 1, 2, 3, 2, 24, 40, 1e-20)
    assert f1.correction_name == "correction" and not f1.shared_gated
    assert f2.shared is None and f2.identity_experts == 2
    assert spec.layers[3].ffn is None and spec.layers[3].post_norm is None
    again, _ = config_from_json(cfg.to_json())
    assert again == cfg


def test_config_without_optional_parts():
    cfg, spec = config_from_json(fk.FB)
    m = [l.mixer for l in spec.layers]
    assert [x.value_mix for x in m] == ["source", "mix", "none", "mix"]
    assert m[0].position.scaling is None and m[2].position is None
    assert m[1].keep_first == 6 and m[1].window == 4 and m[3].conv_taps == 1
    f = spec.layers[0].ffn
    assert (f.identity_experts, f.group_count, f.shared) == (0, 0, None)


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "key/value heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rotated entries"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rotated entries"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=-1), "must not be negative"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "cannot be mixed"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "identity experts"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=4), "groups"),
    (lambda c: c["layers"][1]["mixer"].update(heads="6"), "must be an integer"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "'scale' is missing"),
    (lambda c: c["embedding"].pop("bigram"), "'bigram' is missing"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c.pop("width"), "'width' is missing"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_config_refuses_what_it_cannot_run(change, match):
    cfg = copy.deepcopy(fk.FA)
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        config_from_json(cfg)


# -- the plain statement's mechanisms ----------------------------------------------
def test_plain_pair_rows_and_norm():
    assert plain.bigram_rows([4, 7, 7, 0], 10, 3, 5) == [10, (12 + 35) % 10, (21 + 35) % 10, 21 % 10]
    assert plain.bigram_rows([9], 10, 3, 5) == [10]
    assert torch.allclose(plain.rms_div(torch.tensor([[3.0, 4.0]], dtype=D), 0.0),
                          torch.tensor([[3.0, 4.0]], dtype=D) / math.sqrt(12.5))
    z = torch.tensor([0.5, -1.5], dtype=D)
    want = [0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
            for v in (0.5, -1.5)]
    assert torch.allclose(plain.gelu_tanh(z), torch.tensor(want, dtype=D))


def test_plain_convolution_and_both_pairings():
    # taps (oldest .. current) = (100, 10, 1): token t reads u[t-2], u[t-1], u[t]
    u = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=D)
    y = plain.causal_conv(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=D))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0]
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 7.0]]], dtype=D).repeat(2, 1, 1)
    f = [0.5, 0.25]
    a0, a1 = 3 * 0.5, 3 * 0.25
    half = plain.rotate(v, [0, 3], f, 4, False, 2.0)
    assert torch.equal(half[0], v[0] * torch.tensor([2.0, 2.0, 2.0, 2.0, 1.0], dtype=D))
    want = torch.tensor([1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                         3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)],
                        dtype=D) * 2.0
    assert torch.allclose(half[1, 0, :4], want) and half[1, 0, 4] == 7.0
    inter = plain.rotate(v, [0, 3], f, 4, True)
    want = torch.tensor([1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
                         3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1)],
                        dtype=D)
    assert torch.allclose(inter[1, 0, :4], want) and torch.equal(inter[0], v[0])


def test_plain_stretched_frequencies_by_hand():
    # wavelengths 2 pi / f against original / high = 8 and original / low = 32
    f = [1.0, 0.5, 0.1]           # 6.28 (kept), 12.57 (blended), 62.8 (divided)
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
    out = plain.stretched_by_wavelength(f, sc)
    s = (32 / (2 * math.pi / 0.5) - 1.0) / 3.0
    assert out[0] == 1.0 and out[2] == 0.1 / 4.0
    assert math.isclose(out[1], (1 - s) * 0.5 / 4.0 + s * 0.5)
    # the ramp: pair(t) = dims ln(original / (2 pi t)) / (2 ln base)
    dims, base = 8, 100.0
    sc = {"factor": 2.0, "original": 64, "fast": 4.0, "slow": 1.0}
    lo = max(math.floor(dims * math.log(64 / (2 * math.pi * 4)) / (2 * math.log(base))), 0)
    hi = min(math.ceil(dims * math.log(64 / (2 * math.pi * 1)) / (2 * math.log(base))), dims - 1)
    assert (lo, hi) == (0, 3)
    out, mag = plain.stretched_by_ramp(plain.base_frequencies(dims, base), dims, base, sc)
    assert math.isclose(mag, 0.1 * math.log(2.0) + 1.0)
    for i, v in enumerate(out):
        r = min(max(i / 3.0, 0.0), 1.0)
        fi = base ** (-2.0 * i / dims)
        assert math.isclose(v, fi / 2.0 * r + fi * (1 - r))


def test_plain_window_kept_tokens_and_sink():
    assert [j for j in range(9) if plain.visible(8, j, 3, 0)] == [6, 7, 8]
    assert [j for j in range(9) if plain.visible(8, j, 3, 2)] == [0, 1, 6, 7, 8]
    assert [j for j in range(3) if plain.visible(1, j, 3, 2)] == [0, 1]
    # one head, scores 0: the weights are 1 / n, and 1 / (n + 1) with the sink
    q = torch.zeros(4, 1, 2, dtype=D)
    k = torch.zeros(4, 1, 2, dtype=D)
    v = torch.arange(4, dtype=D).reshape(4, 1, 1) + 1.0
    plain_out = plain.attend(q, k, v, 1.0, 2, 0, False)[:, 0].tolist()
    assert plain_out == [1.0, 1.5, 2.5, 3.5]
    sunk = plain.attend(q, k, v, 1.0, 2, 0, True)[:, 0]
    assert torch.allclose(sunk, torch.tensor([0.5, 1.0, 5.0 / 3, 7.0 / 3], dtype=D))
    kept = plain.attend(q, k, v, 1.0, 2, 1, False)[:, 0]
    assert torch.allclose(kept, torch.tensor([1.0, 1.5, 2.0, 8.0 / 3], dtype=D))


def test_plain_choice_of_experts_by_hand():
    s = torch.tensor([0.05, 0.30, 0.10, 0.25, 0.20, 0.10], dtype=D)
    none = torch.zeros(6, dtype=D)
    idx, w = plain.choose(s, none, 2, 1, 1)
    assert idx == [1, 3] and torch.allclose(w, torch.tensor([0.30, 0.25], dtype=D) / 0.55)
    # three groups of two; the best two are (0.30) and (0.25): output 4 cannot be chosen
    idx, w = plain.choose(s, none, 3, 3, 2)
    assert idx == [1, 3, 2]
    # the correction moves the choice, not the weights: negative corrections still order
    corr = torch.tensor([0.0, -1.0, -0.5, -1.0, -0.3, -0.05], dtype=D)
    idx, w = plain.choose(s, corr, 2, 1, 1)
    assert idx == [0, 5] and torch.allclose(w, torch.tensor([0.05, 0.10], dtype=D) / 0.15)
    # a group whose best corrected value is lowest is out although all values are negative
    idx, _ = plain.choose(s, corr - 5.0, 2, 3, 1)
    assert idx == [0, 1]


def test_plain_identity_expert_returns_its_input():
    w = {"m.router": torch.tensor([[0.0], [50.0]], dtype=D), "m.correction": torch.zeros(2, dtype=D),
         "m.e0.gate": torch.ones(1, 1, dtype=D), "m.e0.up": torch.ones(1, 1, dtype=D),
         "m.e0.down": torch.ones(1, 1, dtype=D) * 9.0}
    f = {"router": {"experts": 1, "top": 1, "identity": 1}, "expert": {"ff": 1}}
    h = torch.tensor([[2.0], [-3.0]], dtype=D)
    out = plain.moe_ff(h, w, "m", f)
    silu = lambda z: z / (1.0 + math.exp(-z))
    # a positive input goes to output 1 (identity), a negative one to expert 0
    assert torch.allclose(out[:, 0], torch.tensor([2.0, silu(-3.0) * -3.0 * 9.0], dtype=D))


def test_later_layers_mix_with_the_first_layers_values(tmp_path):
    """Setting a later layer's mixing weight to zero changes the logits; so does changing
    the first layer's own (unused) weight not."""
    d = fk.make_model_dir(fk.FA, tmp_path / "m", 2)
    cfg, w = plain.read_model_folder(d)
    toks = fk.make_requests(fk.FA, [12], 1)["r0"]
    base = plain.forward(cfg, w, toks)
    w2 = dict(w)
    w2["l2.mix.vmix"] = torch.zeros(())
    assert (plain.forward(cfg, w2, toks) - base).abs().max() > 1e-4
    w3 = dict(w)
    w3["l0.mix.vmix"] = torch.ones(()) * 0.9
    assert torch.equal(plain.forward(cfg, w3, toks), base)


# -- the cache manager keeps the first pages of a windowed group ----------------------
def test_pages_of_kept_first_tokens_are_not_given_back():
    mgr = CacheManager([CacheGroup(window=6, layers=(0,), keep_first=5),
                        CacheGroup(window=6, layers=(1,))], 16, 4, 2)
    mgr.open("a")
    assert mgr.reserve("a", 30)
    mgr.advance("a", 30)
    kept, plain_window = mgr.table("a", 0), mgr.table("a", 1)
    # tokens 0..4 live in pages 0 and 1; the window 25..29 (and the next query) in pages 6, 7
    assert [p >= 0 for p in kept] == [True, True, False, False, False, False, True, True]
    assert [p >= 0 for p in plain_window] == [False] * 6 + [True, True]
    mgr.check_invariants()
    mgr.close("a")
    assert mgr.free_pages(0) == 16 and mgr.free_pages(1) == 16


# -- the engine's host logic ---------------------------------------------------------
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, name, cfg, seed, lengths, page, kind):
    d = fk.make_model_dir(cfg, tmp_path / "m", seed)
    reqs = fk.make_requests(cfg, lengths, seed)
    ref = fk.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, "float32", traces.peak_tokens(steps), page_size=page, max_live=4,
                         device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, steps)
    mc.compare(rows, ref, 2e-5, f"{name}/{kind}")
    if kind in ("whole", "tail", "portions"):
        assert len(rows) == sum(lengths)


def test_portions_of_two_tokens_and_single_tokens_agree_with_whole(tmp_path):
    """The same prompt whole, in portions of two and token by token: the previous token,
    the convolutions' kept inputs and the caches carry everything a cut needs."""
    d = fk.make_model_dir(fk.FB, tmp_path / "m", 7)
    toks = fk.make_requests(fk.FB, [27], 3)["r0"]
    ref = fk.reference_rows(d, {"a": toks})
    for size in (2, 1, 3, 5):
        steps = [{"step": i, "entries": [{"id": "a", "tokens": toks[a:a + size],
                                          "want": list(range(len(toks[a:a + size])))}],
                  "end": ["a"] if a + size >= len(toks) else []}
                 for i, a in enumerate(range(0, len(toks), size))]
        sess = ReplaySession(d, "float32", 64, page_size=4, max_live=1, device="cpu",
                             ops=host_ops)
        rows = mc.run_trace(sess, steps)
        assert len(rows) == len(toks)
        mc.compare(rows, ref, 2e-5, f"portions of {size}")


def test_state_slot_of_a_finished_request_starts_anew(tmp_path):
    """Two requests one after the other in a pool with one slot: the second must see
    neither the first one's last token nor the inputs its convolutions kept."""
    d = fk.make_model_dir(fk.FA, tmp_path / "m", 2)
    reqs = fk.make_requests(fk.FA, [12, 9], 5)
    ref = fk.reference_rows(d, reqs)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=1, device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, traces.whole(reqs))
    mc.compare(rows, ref, 2e-5, "slot reuse")


def test_the_previous_token_is_state_of_the_request(tmp_path):
    d = fk.make_model_dir(fk.FA, tmp_path / "m", 1)
    sess = ReplaySession(d, "float32", 128, page_size=4, max_live=2, device="cpu", ops=host_ops)
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": [5, 9, 17], "want": []},
                                          {"id": "b", "tokens": [44], "want": []}], "end": []})
    model, storage = sess.runtime.model, sess.runtime.storage
    unit = model.extra_cache_units[0]
    prev = storage.state[unit]["previous_token"]
    assert int(prev[sess.manager.slot("a"), 0]) == 17 and int(prev[sess.manager.slot("b"), 0]) == 44
    conv = storage.state[0]["attention_conv_inputs"]
    assert conv.shape[1] == 2 and conv[sess.manager.slot("a")].abs().max() > 0
    assert "attention_conv_inputs" not in storage.state.get(1, {})


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = fk.make_model_dir(fk.FB, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(fk.make_requests(fk.FB, [7, 19, 3], 8).values())
    eng = Engine.create(EngineConfig(model=d, dtype="float32", device="cpu", block_size=4,
                                     max_num_seqs=2, num_gpu_blocks_override=64,
                                     prefill_chunk=5, max_model_len=64), ops=host_ops)
    done = eng.generate([Request(p, SamplingParams(max_tokens=6, ignore_eos=True))
                         for p in prompts])
    for p, c_out in zip(prompts, done):
        seq = list(p)
        for _ in range(6):
            seq.append(int(plain.forward(c, w, seq)[-1].argmax()))
        assert c_out.output_tokens == seq[len(p):]


def test_preemption_rebuilds_state_and_cache(tmp_path):
    """A pool too small for all three requests: the preempted ones give back pages and
    slot, start again from position 0, and generate the same tokens."""
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = fk.make_model_dir(fk.FA, tmp_path / "m", 0)
    reqs = fk.make_requests(fk.FA, [5, 9, 17], 0)

    def run(pages):
        eng = Engine.create(EngineConfig(model=d, dtype="float32", device="cpu", block_size=4,
                                         max_num_seqs=3, num_gpu_blocks_override=pages,
                                         max_model_len=64), ops=host_ops)
        outs = eng.generate([Request(t, SamplingParams(max_tokens=8, ignore_eos=True))
                             for t in reqs.values()])
        return [c.output_tokens for c in outs], eng.stats()["preemptions"]
    roomy, p0 = run(64)
    tight, p1 = run(6)
    assert p0 == 0 and p1 >= 1 and roomy == tight


def test_an_unused_blend_weight_may_be_there_or_not(tmp_path):
    """A layer that mixes nothing has no use for the scalar; a folder runs with it and
    without it, and a scalar that a mixing layer needs is still missed."""
    import os
    from inferx_b200.weights.loader import WeightError
    from inferx_b200.weights.safetensors_io import Checkpoint, write_safetensors
    d = fk.make_model_dir(fk.FA, tmp_path / "m", 3)
    reqs = fk.make_requests(fk.FA, [9, 14], 1)
    ref = fk.reference_rows(d, reqs)

    def rewrite(drop):
        ck = Checkpoint(d)
        kept = {n: ck.get(n).clone() for n in ck.names() if n != drop}
        ck.close()
        write_safetensors(os.path.join(d, "model.safetensors"), kept.items(),
                          metadata={"format": "pt"})

    def replay():
        sess = ReplaySession(d, "float32", 128, page_size=4, max_live=2, device="cpu",
                             ops=host_ops)
        return mc.run_trace(sess, traces.whole(reqs))
    mc.compare(replay(), ref, 2e-5, "with the unused scalar")
    rewrite("l3.mix.vmix")
    mc.compare(replay(), ref, 2e-5, "without the unused scalar")
    rewrite("l2.mix.vmix")
    with pytest.raises(WeightError, match="l2.mix.vmix"):
        replay()
