"""Revelix without a GPU: the configuration reader, the blueprint, the cache's share (states per slot, a window that
keeps the first positions), and the plain implementation's mechanisms against closed forms."""

import copy
import math

import pytest
import torch
import torch.nn.functional as F

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.cache.paged import KVGroupSpec, PagedCache
from flashdecode_cuda_b200.config import ConfigError, load_config
from flashdecode_cuda_b200.engine.model import Model
from flashdecode_cuda_b200.parts.rope import RotaryScaled
from revelix_helpers import REVELIX, random_config
from plain import revelix_plain as P


# ---------------------------------------------------------------- configuration
@pytest.mark.parametrize("name", sorted(REVELIX))
def test_config_round_trip(name):
    cfg = load_config(REVELIX[name])
    assert cfg.architecture == "Revelix"
    again = load_config(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    raw = REVELIX[name]
    assert [L.type for L in cfg.layers] == [L["type"] for L in raw["layers"]]
    assert cfg.vocab == raw["vocab"] and cfg.width == raw["width"] and cfg.norm_eps == raw["norm"]["eps"]
    assert cfg.logit_scale == raw.get("logit_scale", 1.0)


def test_configurations_drawn_at_random_round_trip():
    for seed in range(40):
        raw = random_config(seed)
        cfg = load_config(raw)
        assert load_config(cfg.to_dict()).to_dict() == cfg.to_dict()
        m = Model.from_config(cfg, torch.float32, "cpu")
        names = [s.name for s in m.tensor_specs()]
        assert len(names) == len(set(names))


def test_what_a_file_leaves_out():
    cfg = load_config(REVELIX["Q"])
    par = cfg.layers[1].mixer
    assert par.left_scale == par.right_scale == 1.0 and cfg.logit_scale == 1.0
    assert par.left.softcap is None and par.left.rot is None and par.left.keep_first == 0 and par.left.window == 16
    assert cfg.layers[0].mixer.rot is None
    no_window = load_config(REVELIX["R"]).layers[2].mixer.left
    assert no_window.window is None and no_window.keep_first == 0
    assert "mask" not in load_config(REVELIX["R"]).to_dict()["layers"][2]["mixer"]["left"]


def test_config_errors_name_the_place():
    bad = copy.deepcopy(REVELIX["P"])
    del bad["layers"][0]["mixer"]["right"]["vdim"]
    with pytest.raises(ConfigError, match=r"layers\[0\]\.mixer\.right misses 'vdim'"):
        load_config(bad)
    bad = copy.deepcopy(REVELIX["P"])
    bad["layers"][1]["mixer"]["decay"] = [0.9, 0.9]
    with pytest.raises(ConfigError, match="one number per head"):
        load_config(bad)
    bad = copy.deepcopy(REVELIX["P"])
    bad["layers"][0]["type"] = "attention"
    with pytest.raises(ConfigError, match="mixers are"):
        load_config(bad)
    bad = copy.deepcopy(REVELIX["P"])
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 4
    with pytest.raises(ConfigError, match="multiple of"):
        load_config(bad)
    bad = copy.deepcopy(REVELIX["P"])
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 34
    with pytest.raises(ConfigError, match="dims"):
        load_config(bad)
    bad = copy.deepcopy(REVELIX["P"])
    bad["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(ConfigError, match="dense"):
        load_config(bad)
    odd = copy.deepcopy(REVELIX["P"])
    odd["layers"][1]["mixer"]["gate"] = "swish"
    with pytest.warns(UserWarning, match="does not define"):
        cfg = load_config(odd)
    assert cfg.unknown_keys == ["layers[1].mixer.gate"]
    assert cfg.to_dict() == load_config(REVELIX["P"]).to_dict()


# ---------------------------------------------------------------- blueprint and cache layout
def test_blueprint_declares_the_tensors_and_what_every_layer_keeps():
    m = Model.from_config(load_config(REVELIX["P"]), torch.float32, "cpu")
    spec = {s.name: s for s in m.tensor_specs()}
    assert {"embed", "final.norm", "final.norm.b", "final.norm.alpha", "l0.norm1.alpha", "l0.mix.left.q.b",
            "l0.mix.left.k.conv", "l0.mix.left.sink", "l0.mix.left.talk", "l0.mix.right.lower", "l0.mix.right.f.b",
            "l0.mix.right.norm", "l0.mlp.act", "l1.mix.g", "l1.mlp.down", "l1.norm2.b"} <= set(spec)
    assert not any(n.startswith("head") for n in spec)                       # the logits come from the embedding table
    assert spec["l0.mix.left.q"].shape == (6 * 32, 96) and spec["l0.mix.left.v"].shape == (2 * 40, 96)
    assert spec["l0.mix.left.q.conv"].shape == (6 * 32, 4) and spec["l0.mix.left.talk"].shape == (6, 6)
    assert spec["l0.mix.right.f"].shape == (3 * 24, 96) and spec["l0.mix.right.norm"].shape == (16,)
    assert spec["l0.mix.left.o"].shape == (96, 6 * 40) and spec["l0.mix.right.o"].shape == (96, 3 * 16)
    assert spec["l1.mix.q"].shape == (4 * 24, 96) and spec["l1.mix.o"].shape == (96, 4 * 40)
    assert spec["l0.norm1.alpha"].shape == () and spec["l0.mlp.act"].shape == (2,)
    groups = m.cache_groups()
    assert [(g.n_layers, g.n_kv_heads, g.head_dim, g.value_dim, g.window, g.keep_first) for g in groups] == [(1, 2, 32, 40, 27, 5)]
    q = Model.from_config(load_config(REVELIX["Q"]), torch.float32, "cpu")
    assert "l1.norm2" not in {s.name for s in q.tensor_specs() if not s.optional}       # no feed-forward, no second norm
    assert [(g.n_layers, g.window, g.keep_first) for g in q.cache_groups()] == [(2, 16, 0)]
    r = Model.from_config(load_config(REVELIX["R"]), torch.float32, "cpu")
    assert sorted((g.window or 0, g.keep_first) for g in r.cache_groups()) == [(0, 0), (9, 14)]


def test_states_per_slot_are_zeroed_at_admission():
    m = Model.from_config(load_config(REVELIX["P"]), torch.float32, "cpu")
    groups, states, runs = m._cache_layout()
    # layer 0: the last three projected values of the convolved channels and the recurrence's matrix; layer 1: retention's
    shapes = {s.name: tuple(s.shape) for s in states}
    assert shapes == {"run0.left.conv": (3, (6 + 2) * 32 + 2 * 40), "run0.right.state": (3, 24, 16),
                      "run1.state": (4, 24, 40)}
    assert all(s.dtype == torch.float32 for s in states)
    assert [r[0] for r in runs] == [0, None] and runs[1][3] == {"state": "run1.state"}
    c = PagedCache(groups, states, num_blocks=8, max_slots=2, max_blocks_per_seq=4, block_size=4, dtype=torch.float32,
                   device="cpu")
    a = c.admit()
    b = c.admit()
    for st in c.states.values():
        st[a] += 3.0
        st[b] += 5.0
    c.release(a)
    again = c.admit()                                     # the freed slot, used again
    assert again == a
    assert all(float(st[a].abs().max()) == 0.0 and float(st[b].min()) == 5.0 for st in c.states.values())


def test_a_window_that_keeps_the_first_positions_gives_back_only_the_middle():
    c = PagedCache([KVGroupSpec(1, 1, 8, 6, None, None, False, 5)], [], num_blocks=16, max_slots=2,
                   max_blocks_per_seq=16, block_size=4, dtype=torch.float32, device="cpu")
    s = c.admit()
    c.reserve([(s, 30)]); c.advance(s, 30)
    # the next query (30) sees 25..30 and 0..4: blocks 0 and 1 (positions 0..7) stay, blocks of 8..23 go, 24.. stay
    blocks = c.slots[s].blocks[0]
    assert [b >= 0 for b in blocks[:8]] == [True, True, False, False, False, False, True, True]
    assert c.blocks_in_use() == [4]
    c.check_invariants()
    c.release(s)
    assert c.blocks_in_use() == [0]


# ---------------------------------------------------------------- the plain mechanisms
def test_plain_norm_computes_no_mean_and_no_variance():
    x = torch.tensor([[0.5, -2.0, 100.0]], dtype=torch.float64)
    w, b = torch.tensor([2.0, 1.0, 3.0]).double(), torch.tensor([0.1, 0.0, -1.0]).double()
    y = P.dyn_tanh(x, w, b, torch.tensor(0.5).double())
    assert torch.allclose(y, torch.tensor([[2 * math.tanh(0.25) + 0.1, math.tanh(-1.0), 3.0 - 1.0]]).double())
    y2 = P.dyn_tanh(torch.tensor([[0.5, 7.0, -3.0]]).double(), w, b, torch.tensor(0.5).double())
    assert y2[0, 0] == y[0, 0]                                   # an element's output does not depend on its neighbours


def test_plain_rotation_pairs_and_stretched_frequencies():
    x = torch.zeros(1, 1, 8, dtype=torch.float64)
    x[0, 0, 0] = 1.0
    f = torch.tensor([math.pi / 2, 0.1], dtype=torch.float64)
    half = P.rotate(x, torch.tensor([1]), 4, f, 1.0, interleaved=False)
    pairs = P.rotate(x, torch.tensor([1]), 4, f, 1.0, interleaved=True)
    assert torch.allclose(half[0, 0], torch.tensor([0, 0, 1.0, 0, 0, 0, 0, 0]).double(), atol=1e-12)     # (0, 2) is a pair
    assert torch.allclose(pairs[0, 0], torch.tensor([0, 1.0, 0, 0, 0, 0, 0, 0]).double(), atol=1e-12)    # (0, 1) is a pair
    x[0, 0, 5] = 3.0
    assert float(P.rotate(x, torch.tensor([9]), 4, f, 1.0, interleaved=True)[0, 0, 5]) == 3.0             # beyond dims: untouched
    # frequencies: the fastest pair keeps its own, the slowest is divided by the factor, cos and sin grow
    fr, mag = P.rot_frequencies(48, 1e6, {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0})
    plain, one = P.rot_frequencies(48, 1e6)
    assert one == 1.0 and abs(mag - (0.1 * math.log(8.0) + 1)) < 1e-12
    assert fr[0] == plain[0] and abs(float(fr[-1] / plain[-1]) - 1 / 8) < 1e-12
    assert bool((fr[1:] <= fr[:-1]).all())
    lo = max(math.floor(48 * math.log(1024 / (2 * math.pi * 32.0)) / (2 * math.log(1e6))), 0)
    hi = min(math.ceil(48 * math.log(1024 / (2 * math.pi * 1.0)) / (2 * math.log(1e6))), 47)
    assert bool((fr[:lo + 1] == plain[:lo + 1]).all()) and torch.allclose(fr[hi:], plain[hi:] / 8)
    # the product's tables come from the same frequencies
    pos = RotaryScaled(48, 1e6, {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0})
    got, got_mag = pos.frequencies()
    assert torch.allclose(got, fr, rtol=1e-13, atol=0) and got_mag == mag


def test_plain_short_conv_is_causal_and_ordered():
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)            # the last tap meets the newest value
    assert P.short_conv(u, w)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]


def test_plain_recurrences_against_their_sums():
    torch.manual_seed(0)
    S, H, d, dv = 7, 2, 3, 4
    q, k, v = torch.randn(S, H, d).double(), torch.randn(S, H, d).double(), torch.randn(S, H, dv).double()
    decay = [0.5, 1.0]
    o = P.decayed_recurrence(q, k, v, decay)
    for h in range(H):
        for t in range(S):
            want = sum(decay[h] ** (t - j) * float(q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(o[t, h], want)
    f = torch.rand(S, H, d).double()
    o = P.gated_recurrence(q, f, v)
    for t in (0, 3, 6):
        want = torch.zeros(H, dv).double()
        for j in range(t + 1):
            keep = torch.ones(H, d).double()
            for m in range(j + 1, t + 1):
                keep = keep * f[m]
            want += torch.einsum("hd,hv->hv", q[t] * keep * (1 - f[j]), v[j])
        assert torch.allclose(o[t], want)
    # a gate of one keeps the state as it was; a gate of zero replaces it by the newest value
    ones = P.gated_recurrence(q, torch.ones(S, H, d).double(), v)
    assert float(ones.abs().max()) == 0.0
    zeros = P.gated_recurrence(q, torch.zeros(S, H, d).double(), v)
    assert torch.allclose(zeros, q.sum(-1, keepdim=True) * v)


def test_plain_window_keeps_the_first_positions():
    vis = [[P.window_visible(i, j, 3, 2) for j in range(8)] for i in range(8)]
    assert [j for j in range(8) if vis[7][j]] == [0, 1, 5, 6, 7]
    assert [j for j in range(8) if vis[2][j]] == [0, 1, 2]
    assert [j for j in range(8) if vis[4][j]] == [0, 1, 2, 3, 4]
    S, H, d = 8, 1, 2
    q, k = torch.zeros(S, H, d).double(), torch.zeros(S, H, d).double()
    v = torch.eye(S).double()[:, None, :]                                  # value j marks position j
    out = P.mixed_head_attention(q, k, v, 1.0, None, 3, 2, torch.tensor([-1e9]).double(), torch.ones(1, 1).double())
    assert torch.allclose(out[7, 0], torch.tensor([1, 1, 0, 0, 0, 1, 1, 1.0]).double() / 5)


def test_plain_sink_cap_and_mixed_heads():
    S, H, d, dv = 1, 2, 2, 3
    q, k = torch.zeros(S, H, d).double(), torch.zeros(S, 1, d).double()
    v = torch.ones(S, 1, dv).double()
    sink = torch.tensor([0.0, math.log(3.0)]).double()
    eye = torch.eye(2).double()
    out = P.mixed_head_attention(q, k, v, 1.0, None, None, 0, sink, eye)
    assert torch.allclose(out[0, 0], torch.full((dv,), 0.5).double()) and torch.allclose(out[0, 1], torch.full((dv,), 0.25).double())
    swap = torch.tensor([[0.0, 1.0], [2.0, 0.0]]).double()               # head 0 takes head 1's weights; head 1 twice head 0's
    out = P.mixed_head_attention(q, k, v, 1.0, None, None, 0, sink, swap)
    assert torch.allclose(out[0, 0], torch.full((dv,), 0.25).double()) and torch.allclose(out[0, 1], torch.full((dv,), 1.0).double())
    # a cap of c bounds every score by c: two keys whose scores are +1000 and -1000 weigh e^c : e^-c
    q2 = torch.tensor([[[1000.0, 0.0]]]).double().expand(2, 1, 2).contiguous()
    k2 = torch.tensor([[[1.0, 0.0]], [[-1.0, 0.0]]]).double()
    v2 = torch.tensor([[[1.0]], [[0.0]]]).double()
    out = P.mixed_head_attention(q2, k2, v2, 1.0, 2.0, None, 0, torch.tensor([-1e9]).double(), torch.ones(1, 1).double())
    assert abs(float(out[1, 0, 0]) - math.exp(2) / (math.exp(2) + math.exp(-2))) < 1e-9


def test_plain_activation_is_smooth_at_zero_and_quadratic_above():
    p, q = torch.tensor(0.3).double(), torch.tensor(-0.2).double()
    z = torch.tensor([-1e-7, 0.0, 1e-7, 2.0, -50.0]).double()
    y = P.two_branch_act(z, p, q)
    assert abs(float(y[0])) < 1e-6 and float(y[1]) == 0.0 and abs(float(y[2])) < 1e-6
    assert abs(float(y[3]) - (float(F.softplus(p)) * 4 + 1.0)) < 1e-12
    assert abs(float(y[4]) - ((0.5 + float(F.softplus(q))) * (math.exp(-50) - 1 + 50) - 25)) < 1e-9


def test_random_model_folder_round_trip(tmp_path):
    folder = fd.write_random_model(tmp_path / "m", REVELIX["R"], seed=3)
    assert load_config(folder).to_dict() == load_config(REVELIX["R"]).to_dict()
    w = fd.weights.load_checkpoint(folder)
    assert w["l0.mix.q"].shape == (2 * 136, 72) and w["l1.mix.left.k.conv"].shape == (3 * 24, 2)
    assert w["l1.mix.right.lower"].shape == (16,) and 0 < float(w["l1.mix.right.lower"].float().min())
    assert float(w["l1.mix.right.lower"].float().max()) < 1 and w["l2.mix.left.sink"].shape == (2,)
    assert "l2.mlp.up" not in w and "l0.norm2" not in w
    logits = P.forward(REVELIX["R"], w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 160) and bool(torch.isfinite(logits).all())
