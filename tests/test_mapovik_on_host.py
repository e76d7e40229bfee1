"""The Mapovik design on the CPU: its configuration reader, the plain statement's own
mechanisms on values computed by hand, and the engine's host logic (state slots, caches
per pass, pages, batching) with the kernels replaced by their plain statements
(tests/host_ops.py)."""
import copy
import json
import math

import pytest
import torch

import host_ops
import mapovik_cases as mk
import model_cases as mc
import plain_mapovik as plain
import traces
from inferx_b200.config.model_config import ConfigError
from inferx_b200.config.registry import config_from_json
from inferx_b200.engine.replay import ReplaySession

CASES = [("MA", mk.MA, 0, [5, 9, 17, 40, 3, 70], 4), ("MB", mk.MB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("MC", mk.MC, 3, [21, 1, 50, 2, 37], 4)]
D = torch.float64


# -- configuration ---------------------------------------------------------------
def test_config_reads_every_size_and_constant():
    cfg, spec = config_from_json(mk.MA)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.residual_mult, cfg.logit_scale) == \
        (200, 96, 1e-6, 0.5, 2.0)
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (0, 2, 3)
    pair, d1, d2 = (l.mixer for l in spec.layers)
    a, s = pair.left, pair.right
    assert (a.heads, a.kv_heads, a.head_dim, a.value_dim, a.scale, a.window) == \
        (4, 2, 20, 28, 0.3, 0)
    assert (a.position.rotary_dim, a.position.theta, a.position.scaling_factor) == \
        (10, 5000.0, 3.0)
    assert a.fp32_weights and not a.qkv_bias
    assert (s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups) == (3, 8, 12, 1, 4, 3)
    assert (d1.heads, d1.kv_heads, d1.dim, d1.vdim, d1.conv) == (4, 2, 12, 20, 3)
    assert (d2.heads, d2.kv_heads, d2.dim, d2.vdim, d2.conv, d2.unit_eps) == (2, 2, 16, 8, 4, 1e-6)
    f0, f1 = spec.layers[0].ffn, spec.layers[1].ffn
    assert f0.kind == "relu_squared" and f0.intermediate == 72
    assert (f1.kind, f1.num_experts, f1.top_k, f1.expert_intermediate, f1.vocab) == \
        ("moe_table", 5, 2, 24, 200)
    assert spec.layers[2].ffn is None and spec.layers[2].post_norm is None
    assert all(l.residual_scale == 0.5 and l.input_norm.kind == "layernorm" for l in spec.layers)
    # layers 0 and 1 three times, each pass with a cache of its own, then layer 2
    assert [(e.layer, e.cache_copy) for e in spec.schedule] == \
        [(0, 0), (1, 0), (0, 1), (1, 1), (0, 2), (1, 2), (2, 0)]
    befores = [e.before for e in spec.schedule]
    assert [b is not None for b in befores] == [True, False, True, False, True, False, False]
    assert [(b.row, b.project, b.embedding) for b in befores if b] == \
        [(0, "loop.in", False), (1, "loop.in", False), (2, "loop.in", False)]
    assert spec.logit_scale == 2.0 and not spec.tied_head
    again, _ = config_from_json(cfg.to_json())
    assert again == cfg


def test_config_without_optional_parts():
    cfg, spec = config_from_json(mk.MB)
    assert not cfg.has_loop and all(e.before is None and e.cache_copy == 0 for e in spec.schedule)
    full, bare = spec.layers[1].mixer.left, spec.layers[2].mixer.left
    assert full.position.rotary_dim == full.head_dim and full.position.scaling_factor == 1.0
    assert full.value_dim == 0 and full.kv_heads == full.heads
    assert bare.position is None and bare.value_dim == 8
    assert spec.layers[2].ffn is None and spec.logit_scale == 1.0
    assert spec.layers[0].residual_scale == 1.0


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "key/value heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rotated entries"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=22), "rotated entries"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(groups=2), "groups"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=5), "norm groups"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "query/key heads"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "of 5 experts"),
    (lambda c: c["loop"].update(stop=4), "does not fit"),
    (lambda c: c["layers"][1]["mixer"].update(heads="4"), "must be an integer"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "'scale' is missing"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "'right' is missing"),
    (lambda c: c.pop("width"), "'width' is missing"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_config_refuses_what_it_cannot_run(change, match):
    cfg = copy.deepcopy(mk.MA)
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        config_from_json(cfg)


def test_low_rank_sizes_come_from_the_checkpoint(tmp_path):
    """A configuration that does not state the inner sizes of the decay's and the gate's
    low-rank products runs with whatever the folder's tensors have."""
    d = mk.make_model_dir(mk.MA, tmp_path / "m", 5)
    cfg, w = plain.read_model_folder(d)
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)
        layer["mixer"].pop("gate_rank", None)
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    reqs = mk.make_requests(mk.MA, [11], 2)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=1, device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, traces.whole(reqs))
    mc.compare(rows, mk.reference_rows(d, reqs), 2e-5, "ranks from the tensors")


# -- the plain statement's mechanisms ----------------------------------------------
def test_plain_norm_convolution_and_rotation():
    x = torch.tensor([[1.0, 3.0]], dtype=D)
    # mean 2, deviations -1 and 1, variance 1
    out = plain.layer_norm(x, torch.tensor([2.0, 0.5], dtype=D), 0.0)
    assert torch.allclose(out, torch.tensor([[-2.0, 0.5]], dtype=D))
    assert torch.allclose(plain.rms_div(torch.tensor([[3.0, 4.0]], dtype=D), 0.0),
                          torch.tensor([[3.0, 4.0]], dtype=D) / math.sqrt(12.5))
    # taps (oldest .. current) = (100, 10, 1): token t reads x[t-2], x[t-1], x[t]
    xs = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=D)
    y = plain.causal_conv(xs, torch.tensor([[100.0, 10.0, 1.0]], dtype=D),
                          torch.tensor([0.5], dtype=D))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5]
    # entry i turns with entry i + dims/2; what lies beyond dims passes; the factor divides
    # the angle
    v = torch.tensor([[[1.0, 2.0, 0.0, 0.0, 7.0]]], dtype=D).repeat(2, 1, 1)
    pos = torch.tensor([0, 3])
    r = plain.rotate_half(v, pos, 4, 100.0, 2.0)
    assert torch.equal(r[0], v[0])
    a0, a1 = 3 * 1.0 / 2.0, 3 * 100.0 ** -0.5 / 2.0
    want = torch.tensor([math.cos(a0), 2 * math.cos(a1), math.sin(a0), 2 * math.sin(a1), 7.0],
                        dtype=D)
    assert torch.allclose(r[1, 0], want)


def test_plain_state_space_by_hand():
    """One head, one state entry, one value channel, a convolution of one tap: scalars."""
    one = torch.ones(1, 1, dtype=D)
    # rows of the input projection: z, x, B, C, dt
    w = {"p.in": torch.tensor([[1.0], [1.0], [1.0], [1.0], [0.0]], dtype=D),
         "p.conv": torch.ones(3, 1, dtype=D), "p.conv.b": torch.zeros(3, dtype=D),
         "p.dt_bias": torch.tensor([0.3], dtype=D), "p.A_log": torch.tensor([-0.2], dtype=D),
         "p.D": torch.tensor([2.0], dtype=D), "p.norm": torch.ones(1, dtype=D), "p.o": one}
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    hs = [1.0, -0.5, 2.0]
    out = plain.state_space(torch.tensor(hs, dtype=D)[:, None], w, "p", m, 0.0)
    silu = lambda z: z / (1.0 + math.exp(-z))
    dt = math.log1p(math.exp(0.3))
    a = math.exp(-math.exp(-0.2) * dt)
    S, ys = 0.0, []
    for h in hs:
        x = silu(h)
        S = a * S + dt * x * x
        ys.append((S * x + 2.0 * x) * silu(h))
    # one channel: the RMS norm leaves the sign
    assert [float(v) for v in out[:, 0]] == [math.copysign(1.0, y) for y in ys]
    # with a gain and two channels the magnitudes show: check y before the norm through eps
    big = plain.state_space(torch.tensor(hs, dtype=D)[:, None], w, "p", m, 1e12)
    assert torch.allclose(big[:, 0] * 1e6, torch.tensor(ys, dtype=D), rtol=1e-6)


def test_plain_delta_rule_by_hand():
    """One head, one key channel, one value channel.  k is a unit vector, so S^T k is S,
    u = beta (v - g S) and S <- g S + u: a decayed value moved towards v by beta."""
    one = torch.ones(1, 1, dtype=D)
    w = {"p.q": one, "p.k": one, "p.v": one * 3.0, "p.q.conv": one, "p.k.conv": one,
         "p.v.conv": one, "p.b": one * 0.0, "p.a1": one, "p.a2": one * 0.0,
         "p.dt_bias": torch.tensor([0.1], dtype=D), "p.A_log": torch.tensor([0.4], dtype=D),
         "p.norm": torch.ones(1, dtype=D), "p.g1": one, "p.g2": one * 0.0, "p.o": one}
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 1}
    hs = [1.0, 2.0, 0.5]
    out = plain.channel_delta(torch.tensor(hs, dtype=D)[:, None], w, "p", m, 1e12)
    silu = lambda z: z / (1.0 + math.exp(-z))
    g = math.exp(-math.exp(0.4) * math.log1p(math.exp(0.1)))
    S, os_ = 0.0, []
    for h in hs:
        unit = silu(h) / math.sqrt(silu(h) ** 2 + 1e-6)
        S = g * S
        u = 0.5 * (silu(3.0 * h) - S * unit)
        S = S + unit * u
        os_.append(S * unit)            # q scale 1^(-1/2)
    # eps 1e12 turns the norm into a division by 1e6; the gate is sigmoid(0)
    assert torch.allclose(out[:, 0] * 1e6 / 0.5, torch.tensor(os_, dtype=D), rtol=1e-6)


def test_plain_table_picks_experts_by_token_id():
    w = {"m.table": torch.tensor([[0, 1], [1, 0], [1, 2]], dtype=torch.int32)}
    for e, f in enumerate((1.0, 2.0, 4.0)):
        w.update({f"m.e{e}.gate": torch.ones(1, 1, dtype=D), f"m.e{e}.up": torch.ones(1, 1, dtype=D),
                  f"m.e{e}.down": torch.ones(1, 1, dtype=D) * f})
    h = torch.ones(3, 1, dtype=D)
    unit = 1.0 / (1.0 + math.exp(-1.0))
    out = plain.table_experts(h, w, "m", [0, 1, 2])
    assert torch.allclose(out[:, 0], torch.tensor([1.5, 1.5, 3.0], dtype=D) * unit)
    assert torch.allclose(plain.dense_ff(torch.tensor([[2.0], [-2.0]], dtype=D),
                                         {"f.up": torch.ones(1, 1, dtype=D),
                                          "f.down": torch.ones(1, 1, dtype=D) * 3.0}, "f")[:, 0],
                          torch.tensor([12.0, 0.0], dtype=D))


def test_plain_order_of_runs():
    assert plain.run_order(mk.MC) == [(0, None, False), (1, 0, True), (1, 1, True),
                                      (2, None, False)]
    assert plain.run_order(mk.MB) == [(0, None, False), (1, None, False), (2, None, False)]
    assert [f for _, _, f in plain.run_order(mk.MA)] == [True, False] * 3 + [False]


def test_stream_projection_reads_the_embedding_output_in_every_pass(tmp_path):
    """Zeroing the half of the projection that reads the embedding output changes the
    logits; so does zeroing one pass's row of the added table - each is really used."""
    d = mk.make_model_dir(mk.MC, tmp_path / "m", 2)
    cfg, w = plain.read_model_folder(d)
    toks = mk.make_requests(mk.MC, [6], 1)["r0"]
    base = plain.forward(cfg, w, toks)
    w2 = dict(w)
    w2["loop.in"] = w["loop.in"].clone()
    w2["loop.in"][:, cfg["width"]:] = 0
    assert (plain.forward(cfg, w2, toks) - base).abs().max() > 1e-3
    w3 = dict(w)
    w3["loop.step"] = w["loop.step"].clone()
    w3["loop.step"][1] = 0
    assert (plain.forward(cfg, w3, toks) - base).abs().max() > 1e-3


def test_each_pass_of_a_loop_keeps_a_state_of_its_own(tmp_path):
    d = mk.make_model_dir(mk.MC, tmp_path / "m", 1)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=2, device="cpu", ops=host_ops)
    toks = mk.make_requests(mk.MC, [9], 0)["r0"]
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": []})
    model, storage = sess.runtime.model, sess.runtime.storage
    assert model.cache_units == [(0, 0), (1, 0), (2, 0), (1, 1)]
    slot = sess.manager.slot("a")
    first, second = (storage.state[u]["ssd_state"][slot] for u in (1, 3))
    assert first.abs().max() > 0 and second.abs().max() > 0 and not torch.equal(first, second)
    conv_a, conv_b = (storage.state[u]["ssd_conv_inputs"][slot] for u in (1, 3))
    assert conv_a.abs().max() > 0 and not torch.equal(conv_a, conv_b)
    # the delta layers: a convolution of one tap keeps no inputs, four taps keep three
    assert "delta_conv_inputs" not in storage.state[0]
    assert storage.state[2]["delta_conv_inputs"].shape[1] == 3


# -- the engine's host logic ---------------------------------------------------------
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, name, cfg, seed, lengths, page, kind):
    d = mk.make_model_dir(cfg, tmp_path / "m", seed)
    reqs = mk.make_requests(cfg, lengths, seed)
    ref = mk.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, "float32", traces.peak_tokens(steps), page_size=page, max_live=4,
                         device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, steps)
    mc.compare(rows, ref, 2e-5, f"{name}/{kind}")
    if kind in ("whole", "tail", "portions"):
        assert len(rows) == sum(lengths)


def test_portions_of_two_tokens_and_single_tokens_agree_with_whole(tmp_path):
    """The same prompt whole, in portions of two and token by token: the convolutions'
    kept inputs, the states and the caches carry everything a cut needs."""
    d = mk.make_model_dir(mk.MA, tmp_path / "m", 7)
    toks = mk.make_requests(mk.MA, [23], 3)["r0"]
    ref = mk.reference_rows(d, {"a": toks})
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


def test_state_slot_of_a_finished_request_starts_from_zero(tmp_path):
    """Two requests one after the other in a pool with one slot: the second must see
    neither the first one's states nor the inputs its convolutions kept."""
    d = mk.make_model_dir(mk.MA, tmp_path / "m", 2)
    reqs = mk.make_requests(mk.MA, [12, 9], 5)
    ref = mk.reference_rows(d, reqs)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=1, device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, traces.whole(reqs))
    mc.compare(rows, ref, 2e-5, "slot reuse")


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = mk.make_model_dir(mk.MB, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(mk.make_requests(mk.MB, [7, 19, 3], 8).values())
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
    slot, start again from position 0 in a zeroed slot, and generate the same tokens."""
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = mk.make_model_dir(mk.MA, tmp_path / "m", 0)
    reqs = mk.make_requests(mk.MA, [5, 9, 17], 0)

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
