"""Botusun without a GPU: configuration, blueprint, weights' checks, the rotation tables, and the plain
implementation's mechanisms against closed forms."""

import math
import warnings

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.config import ConfigError, load_config
from flashdecode_cuda_b200.config.botusun import BotusunConfig
from flashdecode_cuda_b200.engine.model import Model
from flashdecode_cuda_b200.parts.rope import RotaryScaled
from flashdecode_cuda_b200.weights import WeightError, check
import botusun_helpers as BH
from botusun_helpers import BOTUSUN, random_config
from plain import botusun_plain as P


@pytest.mark.parametrize("name", sorted(BOTUSUN))
def test_configuration_round_trip(name):
    cfg = load_config(BOTUSUN[name])
    assert isinstance(cfg, BotusunConfig) and cfg.architecture == "Botusun"
    again = load_config(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    assert not cfg.unknown_keys


def test_keys_left_out_take_their_neutral_values():
    raw = BH.model(50, 32, 1e-5, [BH.attention(2, 2, 16, 1, 0.25, mlp=BH.moe(4, 2, 8))])
    del raw["layers"][0]["mixer"]["kv_heads"], raw["layers"][0]["mixer"]["conv"], raw["layers"][0]["mixer"]["vdim"]
    cfg = load_config(raw)
    m, f = cfg.layers[0].mixer, cfg.layers[0].mlp
    assert (m.kv_heads, m.conv, m.vdim, m.window, m.rot) == (2, 1, 16, None, None)
    assert (f.groups, f.keep, f.scale) == (1, 1, 1.0)
    assert (cfg.embedding_scale, cfg.residual_mult, cfg.side_dim, cfg.loop_times) == (1.0, 1.0, 0, 0)


@pytest.mark.parametrize("edit,text", [
    (lambda c: c.pop("width"), "misses 'width'"),
    (lambda c: c["layers"][0].update(type="conv"), "mixers are"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(groups={"count": 3, "keep": 1}), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(groups={"count": 4, "keep": 1}, top=3), "hold at least top"),
    (lambda c: c.update(loop={"start": 1, "stop": 0, "times": 2}), "loop"),
    (lambda c: c["layers"][0]["mixer"].update(rot={"dims": 3, "base": 100.0}), "dims must be even"),
])
def test_configuration_errors_name_their_place(edit, text):
    raw = BH.model(50, 32, 1e-5, [BH.attention(6, 2, 16, 2, 0.25, mlp=BH.moe(8, 2, 8, groups=(4, 2)))])
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        load_config(raw)


def test_unknown_keys_warn_and_change_nothing():
    raw = BH.model(50, 32, 1e-5, [BH.gla(2, 8, 8, 4.0, 4)])
    raw["layers"][0]["mixer"]["surprise"] = 1
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        cfg = load_config(raw)
    assert cfg.unknown_keys == ["layers[0].mixer.surprise"] and len(w) == 1


def test_layer_runs_of_loops():
    for loop, want in [(None, [0, 1, 2, 3]), ((1, 3, 2), [0, 1, 2, 1, 2, 3]), ((0, 4, 2), [0, 1, 2, 3] * 2),
                       ((3, 4, 3), [0, 1, 2, 3, 3, 3]), ((2, 2, 5), [0, 1, 2, 3]), ((0, 1, 1), [0, 1, 2, 3])]:
        raw = BH.model(50, 32, 1e-5, [BH.gla(2, 8, 8, 4.0, 4) for _ in range(4)], loop=loop)
        cfg = load_config(raw)
        runs = cfg.layer_runs()
        assert [i for i, _ in runs] == want
        assert [(i, t) for i, t in P.layer_runs(raw)] == runs
        if loop and loop[1] > loop[0]:
            assert [t for i, t in runs if t is not None] == list(range(loop[2]))


@pytest.mark.parametrize("name", sorted(BOTUSUN))
def test_blueprint_and_the_tensors_it_declares(name):
    cfg = load_config(BOTUSUN[name])
    model = Model.from_config(cfg, torch.float32, "cpu")
    runs = cfg.layer_runs()
    assert [r.layer for r in model.schedule] == [i for i, _ in runs]
    assert [r.before_index for r in model.schedule] == [t for _, t in runs]
    names = {s.name for s in model.tensor_specs()}
    assert {"embed", "final.norm"} <= names and ("loop.step" in names) == bool(cfg.loop_times)
    assert ("side.embed" in names) == bool(cfg.side_dim)
    for i, L in enumerate(cfg.layers):
        assert (f"l{i}.mix.a2.b" in names) == (L.type == "gla") and (f"l{i}.mix.k.norm" in names) == (L.type == "attention")
        assert f"l{i}.mix.v" in names if L.type == "gla" else f"l{i}.mix.v" not in names
        assert (f"l{i}.side.proj" in names) == bool(cfg.side_dim)
    # every run of an attention layer has pages of its own, every run of a recurrent layer a state of its own
    groups, states, per_run = model._layout
    n_att = sum(cfg.layers[i].type == "attention" for i, _ in runs)
    assert sum(g.n_layers for g in groups) == n_att
    n_state = sum(1 for i, _ in runs if cfg.layers[i].type == "gla") + \
        sum(1 for i, _ in runs if cfg.layers[i].type == "attention" and cfg.layers[i].mixer.conv > 1)
    assert len(states) == n_state


def test_a_size_only_the_checkpoint_gives():
    """The rows of the decay's narrow projection are not in the configuration: any number fits, as long as both
    matrices agree at bind; random weights need the key."""
    raw = BH.model(50, 32, 1e-5, [BH.gla(2, 8, 8, 4.0, 4)])
    folder_cfg = load_config(raw)
    model = Model.from_config(folder_cfg, torch.float32, "cpu")
    tensors = fd.random_weights(model, 1)
    del raw["layers"][0]["mixer"]["rank"]
    open_model = Model.from_config(load_config(raw), torch.float32, "cpu")
    check(open_model.tensor_specs(), tensors)
    tensors["l0.mix.a1"] = torch.zeros(7, 32)
    tensors["l0.mix.a2"] = torch.zeros(16, 7)
    check(open_model.tensor_specs(), tensors)
    tensors["l0.mix.a2"] = torch.zeros(15, 7)
    with pytest.raises(WeightError, match="l0.mix.a2"):
        check(open_model.tensor_specs(), tensors)
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        fd.random_weights(open_model, 1)


@pytest.mark.parametrize("dims,base,scaling", [(16, 10000.0, None), (48, 1e6, (8.0, 1.0, 4.0, 1024)),
                                               (8, 100.0, (4.0, 2.0, 8.0, 16)), (32, 500000.0, (4.0, 1.0, 4.0, 1024)),
                                               (2, 50.0, (2.0, 1.0, 1.0, 64))])
def test_rotation_tables_follow_the_wavelength_rule(dims, base, scaling):
    sc = None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))
    f = P.rot_frequencies(dims, base, sc)
    if sc is not None:                      # against the rule itself: kept, divided, or between the two
        for i, fi in enumerate(f.tolist()):
            f0 = base ** (-2.0 * i / dims)
            wl = 2 * math.pi / f0
            if wl < sc["original"] / sc["high"]:
                assert fi == pytest.approx(f0)
            elif wl > sc["original"] / sc["low"]:
                assert fi == pytest.approx(f0 / sc["factor"])
            else:
                assert f0 / sc["factor"] - 1e-12 <= fi <= f0 + 1e-12

    class Rt:
        device = torch.device("cpu")
    pos = RotaryScaled(dims, base, sc)
    got, mag = pos.frequencies()
    assert mag == 1.0 and torch.allclose(got, f, rtol=1e-12, atol=0)
    pos.prepare(300, Rt)
    a = torch.outer(torch.arange(300, dtype=torch.float64), f)
    assert torch.allclose(pos.cos[:300].double(), a.cos(), atol=1e-6) and torch.allclose(pos.sin[:300].double(), a.sin(), atol=1e-6)


# ---------------------------------------------------------------- the plain implementation against closed forms
def test_plain_recurrence_against_its_unrolled_sum():
    torch.manual_seed(0)
    S, H, d, dv = 9, 2, 3, 4
    q, k, a = torch.randn(S, H, d).double(), torch.randn(S, H, d).double(), torch.rand(S, H, d).double()
    v = torch.randn(S, H, dv).double()
    o, _ = P.channel_decay_recurrence(q, k, v, a)
    t = S - 1
    want = torch.zeros(H, dv, dtype=torch.float64)
    for j in range(t + 1):
        decay = torch.ones(H, d, dtype=torch.float64)
        for u in range(j + 1, t + 1):
            decay = decay * a[u]
        want += torch.einsum("hd,hv->hv", q[t] * decay * k[j], v[j])
    assert torch.allclose(o[t], want, atol=1e-12)
    first, state = P.channel_decay_recurrence(q[:4], k[:4], v[:4], a[:4])
    rest, _ = P.channel_decay_recurrence(q[4:], k[4:], v[4:], a[4:], state)
    assert torch.allclose(torch.cat([first, rest]), o, atol=1e-12)


def test_plain_attention_window_and_keyless_term():
    torch.manual_seed(1)
    S, d = 12, 4
    q, k, v = torch.zeros(S, 2, d).double(), torch.randn(S, 1, d).double(), torch.randn(S, 1, d).double()
    o = P.sink_softmax_attention(q, k, v, 1.0, 3)
    # all scores are zero: every visible key and the keyless term weigh 1 / (visible + 1)
    for i in range(S):
        lo = max(0, i - 2)
        assert torch.allclose(o[i, 0], v[lo:i + 1, 0].sum(0) / (i + 1 - lo + 1), atol=1e-12)
        assert torch.allclose(o[i, 0], o[i, 1])
    o1 = P.sink_softmax_attention(q, k, v, 1.0, 1)
    assert torch.allclose(o1[:, 0], v[:, 0] / 2, atol=1e-12)
    full = P.sink_softmax_attention(q, k, v, 1.0, None)
    assert torch.allclose(full[S - 1, 0], v[:, 0].sum(0) / (S + 1), atol=1e-12)


def test_plain_routing_keeps_to_the_best_groups():
    h = torch.eye(4, dtype=torch.float64)
    router = torch.tensor([[4.0, 0, 0, 0], [3.9, 0, 0, 0], [0, 0, 0, 0], [0, 0, 0, 0],
                           [3.0, 0, 0, 0], [-9.0, 0, 0, 0], [0, 0, 0, 0], [0, 0, 0, 0]], dtype=torch.float64)
    rc = {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 1}, "scale": 2.0}
    ids, w = P.route(h[:1], router, torch.zeros(8, dtype=torch.float64), rc)
    assert sorted(ids[0].tolist()) == [0, 1]                       # group 0 has the largest two-score sum
    assert torch.allclose(w[0].sort().values, 2.0 * torch.sigmoid(torch.tensor([3.9, 4.0], dtype=torch.float64)))
    # corrections decide the choice but do not enter the weights; with every choice score negative an expert of a group
    # that is not kept still cannot be chosen
    corr = torch.tensor([-50.0, -50.0, -60.0, -60.0, -40.0, -40.0, -70.0, -70.0], dtype=torch.float64)
    ids, w = P.route(h[:1], router, corr, rc)
    assert sorted(ids[0].tolist()) == [4, 5]
    assert torch.allclose(w[0].sort().values, 2.0 * torch.sigmoid(torch.tensor([-9.0, 3.0], dtype=torch.float64)))


def test_plain_convolution_and_rotation():
    u = torch.arange(10, dtype=torch.float64).reshape(5, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = P.short_conv(u, w)
    assert y[:, 1].tolist() == u[:, 1].tolist()
    assert y[:, 0].tolist() == [0.0, 200.0, 420.0, 642.0, 864.0]
    x = torch.randn(6, 2, 8).double()
    f = P.rot_frequencies(4, 100.0)
    r = P.rotate_half(x, torch.arange(6), 4, f)
    assert torch.equal(r[:, :, 4:], x[:, :, 4:]) and torch.allclose(r[0], x[0])
    assert torch.allclose(r[:, :, :4].pow(2).sum(-1), x[:, :, :4].pow(2).sum(-1))
    a = 3 * f[1]
    assert torch.allclose(r[3, 0, 1], x[3, 0, 1] * torch.cos(a) - x[3, 0, 3] * torch.sin(a))


@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations_are_valid_and_the_plain_model_runs(seed):
    raw = random_config(seed)
    cfg = load_config(raw)
    model = Model.from_config(cfg, torch.float32, "cpu")
    W = fd.random_weights(model, seed)
    check(model.tensor_specs(), W)
    logits, layers = P.forward(cfg.to_dict(), W, [1, 2, 3, 4, 5], return_layers=True)
    assert logits.shape == (5, cfg.vocab) and layers.shape[0] == len(cfg.layer_runs()) and bool(torch.isfinite(logits).all())
    # prefix property: what a position's logits are does not depend on what follows
    assert torch.allclose(P.forward(cfg.to_dict(), W, [1, 2, 3])[2], logits[2], atol=1e-9)
