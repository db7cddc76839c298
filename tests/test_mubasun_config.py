"""Mubasun without a GPU: the configuration (registry, round trip, every broken rule named), the layout and the
checkpoint's tensor names, a random folder, and the plain mechanisms against other ways of writing them."""
import copy
import json
import math

import numpy as np
import pytest
import torch

from plain import mubasun_plain as MP
from quicknn_b200.config import MUBASUN, ConfigError, MubasunConfig, find_architecture, load_config, mubasun_spec
from quicknn_b200.config.mubasun import distance_slopes
from quicknn_b200.parts import FEED_FORWARDS, MIXERS, NORMS, PartSpec, expected_tensors
from quicknn_b200.weights import random_tensors, write_safetensors


def _att(heads, kv, dim, vdim, scale, window=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, experts, identity, top, scale, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


RAW = dict(architecture="Mubasun", vocab=120, width=48, max_positions=96, norm={"eps": 1e-5, "groups": 3},
           initializer_range=0.05, layers=[
               {"type": "attention", "mixer": _att(4, 2, 8, 12, 0.3), "mlp": {"kind": "dense", "ff": 64}},
               {"type": "attention", "mixer": _att(2, 1, 12, 8, 0.25, window=5), "mlp": _moe(16, 5, 2, 3, 1.5, shared=24)},
               {"type": "attention", "mixer": _att(4, 2, 8, 12, 0.3, window=7, kv_from=0), "mlp": None},
               {"type": "attention", "mixer": _att(2, 1, 12, 8, 0.2, kv_from=1), "mlp": _moe(8, 3, 0, 1, 1.0)}])


def test_registry_round_trip_and_layout():
    assert find_architecture({"architecture": "Mubasun"}) is MUBASUN
    cfg = MubasunConfig.from_dict(RAW)
    assert MubasunConfig.from_dict(cfg.to_dict()) == cfg
    assert MubasunConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert (cfg.norm_eps, cfg.norm_groups) == (1e-5, 3)
    spec = mubasun_spec(cfg)
    assert [l.block.kind for l in spec.layers] == ["parallel"] * 4 and [l.mixer.kind for l in spec.layers] == ["attention"] * 4
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 1, False)]
    assert spec.head.norm.kind == "group_rmsnorm" and spec.head.norm.params["groups"] == 3 and not spec.head.tied
    assert spec.embedding.position_tensor == "pos" and spec.embedding.n_positions == 96 and spec.embedding.scale == 1.0
    a0, a1, a2 = (spec.layers[i].mixer.params for i in (0, 1, 2))
    assert a0["window"] is None and a1["window"] == 5 and a2["window"] == 7 and a2["shared_kv"] and not a0["shared_kv"]
    assert a0["qk_norm"] == {"eps": 1e-5, "over": "projection"} and a0["out_gate"] and a0["position"].kind == "none"
    assert a1["distance_slopes"] == (2.0 ** -4, 2.0 ** -8) and len(a0["distance_slopes"]) == 4
    assert spec.layers[0].feed_forward.params["activation"] == "xielu" and spec.layers[2].feed_forward is None
    r = spec.layers[1].feed_forward.params
    assert (r["experts"], r["identity"], r["top"], r["route_scale"], r["score"]) == (5, 2, 3, 1.5, "softmax")
    assert r["correction"] and not r["renormalize"] and r["weight_on"] == "output" and r["shared_gate"]
    assert r["shared"].params["intermediate_size"] == 24 and spec.layers[3].feed_forward.params["shared"] is None
    names = expected_tensors(spec)
    assert names["embed"][0] == (120, 48) and names["pos"][0] == (96, 48) and names["head"][0] == (120, 48)
    assert names["l0.mix.q"][0] == (32, 48) and names["l0.mix.v"][0] == (24, 48) and names["l0.mix.g"][0] == (48, 48)
    assert names["l0.mix.o"][0] == (48, 48) and names["l0.mix.q.norm"][0] == (32,) and names["l0.mix.k.norm"][0] == (16,)
    assert names["l0.mlp.up"][0] == (64, 48) and names["l0.mlp.down"][0] == (48, 64) and names["l0.mlp.act"][0] == (2,)
    assert names["l1.mlp.router"][0] == (7, 48) and names["l1.mlp.correction"][0] == (7,) and "l1.mlp.e5.up" not in names
    assert names["l1.mlp.e4.gate"][0] == (16, 48) and names["l1.mlp.e0.down"][0] == (48, 16)
    assert names["l1.mlp.shared.up"][0] == (24, 48) and names["l1.mlp.shared.sg"][0] == (1, 48)
    assert "l2.mix.k" not in names and "l2.mix.v" not in names and "l2.mix.k.norm" not in names and "l2.mix.q.norm" in names
    assert "l2.mlp.up" not in names and names["l3.mlp.router"][0] == (3, 48) and "l3.mlp.shared.sg" not in names
    assert not any(n.endswith(("norm2", ".b")) for n in names) and names["final.norm"][0] == (48,)
    assert set(n.split(".")[0] for n in names) == {"embed", "pos", "final", "head", "l0", "l1", "l2", "l3"}


def _broken(change):
    raw = copy.deepcopy(RAW)
    change(raw)
    return raw


@pytest.mark.parametrize("change,says", [
    (lambda r: r.pop("max_positions"), "max_positions"),
    (lambda r: r.update(max_positions=0), "max_positions"),
    (lambda r: r["norm"].update(groups=5), "norm.groups"),
    (lambda r: r["norm"].update(eps=0.0), "norm.eps"),
    (lambda r: r["layers"][0].update(type="conv"), "layer type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads do not divide"),
    (lambda r: r["layers"][0]["mixer"].update(scale=0.0), "scale"),
    (lambda r: r["layers"][1]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=1), "differ"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "mlp.kind"),
    (lambda r: r["layers"][0]["mlp"].update(ff=0), "inner width"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=8), "router.top"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(experts=0), "experts >= 1"),
    (lambda r: r["layers"][1]["mlp"]["shared"].update(ff=0), "shared.ff"),
])
def test_every_broken_rule_is_named(change, says):
    with pytest.raises((ConfigError, ValueError, TypeError)) as e:
        MubasunConfig.from_dict(_broken(change))
    assert says in str(e.value), str(e.value)


def test_a_random_folder_loads_by_its_config(tmp_path):
    cfg = MubasunConfig.from_dict(RAW)
    tensors = dict(random_tensors(MUBASUN, cfg, 7, torch.bfloat16))
    assert set(tensors) == set(expected_tensors(mubasun_spec(cfg)))
    assert abs(float(tensors["l0.norm1"].float().mean()) - 1.0) < 0.2 and abs(float(tensors["l1.mlp.correction"].float().mean())) < 0.2
    with open(tmp_path / "config.json", "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    arch, again = load_config(str(tmp_path))
    assert arch is MUBASUN and again == cfg
    plain = MP.PlainMubasun(str(tmp_path))
    z = plain.logits([5, 6, 7, 8, 9, 10, 11])
    assert z.shape == (7, 120) and np.isfinite(z).all()
    assert np.abs(plain.logits([5, 6, 7, 8])[:4] - z[:4]).max() < 1e-9     # a position depends on the tokens before it only
    assert len(plain.residual_stream([1, 2, 3])) == 5


def test_the_slopes_and_the_two_ways_to_write_the_bias():
    assert distance_slopes(4) == (0.25, 0.0625, 0.015625, 0.00390625)
    assert np.allclose(distance_slopes(3), MP.slopes(3)) and len(distance_slopes(1)) == 1 and distance_slopes(1)[0] == 2.0 ** -8
    # without a sink a softmax row does not care whether slope * (i - j) is subtracted or slope * j is added
    rng = np.random.default_rng(0)
    s = rng.normal(size=(6, 6))
    i, j = np.arange(6)[:, None], np.arange(6)[None, :]
    def soft(z):
        z = np.where(j <= i, z, -np.inf)
        e = np.exp(z - z.max(-1, keepdims=True))
        return e / e.sum(-1, keepdims=True)
    assert np.allclose(soft(s - 0.3 * (i - j)), soft(s + 0.3 * j))


def test_the_plain_pieces_against_other_ways_of_writing_them():
    rng = np.random.default_rng(1)
    x, w = rng.normal(size=(5, 12)), rng.normal(size=12)
    got = MP.group_norm(x, w, 3, 1e-5)
    for t in range(5):
        for g in range(3):
            piece = x[t, 4 * g:4 * g + 4]
            assert np.allclose(got[t, 4 * g:4 * g + 4], piece / math.sqrt((piece ** 2).mean() + 1e-5) * w[4 * g:4 * g + 4])
    assert np.allclose(MP.group_norm(x, w, 1, 1e-5), MP.rms_unit(x, 1e-5) * w)
    z = np.array([-30.0, -2.0, -1e-9, 0.0, 1e-9, 0.5, 3.0])
    p, q = 0.3, -0.7
    sp = lambda v: math.log1p(math.exp(v))  # noqa: E731
    want = [sp(p) * v * v + v / 2 if v > 0 else (0.5 + sp(q)) * (math.exp(v) - 1 - v) + v / 2 for v in z]
    assert np.allclose(MP.xielu(z, p, q), want) and MP.xielu(np.zeros(1), p, q)[0] == 0.0
    # the function is continuous at 0 with slope 1/2 on both sides
    assert abs(MP.xielu(np.array([1e-6]), p, q)[0] - 5e-7) < 1e-11 and abs(MP.xielu(np.array([-1e-6]), p, q)[0] + 5e-7) < 1e-11


def test_window_gate_whole_norm_and_shared_keys_in_the_plain_attention():
    rng = np.random.default_rng(3)
    W, m = 8, {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5}
    w = {"q": rng.normal(size=(8, W)), "k": rng.normal(size=(4, W)), "v": rng.normal(size=(6, W)), "o": rng.normal(size=(W, 12)),
         "g": rng.normal(size=(12, W)), "q.norm": rng.normal(size=8), "k.norm": rng.normal(size=4)}
    h = rng.normal(size=(6, W))
    y, kv = MP.attention(h, w, m, 1e-5)
    y2, _ = MP.attention(h, {k: v for k, v in w.items() if k[0] not in "kv"}, m, 1e-5, kv=kv)
    assert np.allclose(y, y2) and kv[0].shape == (6, 4) and kv[1].shape == (6, 6)
    # the norm is over all query heads at once: scaling one head's rows of W_q changes the other head's queries too
    w2 = dict(w, q=np.concatenate([w["q"][:4] * 10, w["q"][4:]]))
    qa = MP.rms_unit(h @ w["q"].T, 1e-5)
    qb = MP.rms_unit(h @ w2["q"].T, 1e-5)
    assert np.abs(qa[:, 4:] - qb[:, 4:]).max() > 0.1 and np.allclose((qb ** 2).mean(-1), 1.0, atol=1e-4)
    # a window of 1: the last position sees itself alone, so its output is its own value, gated, through W_o
    y1, kv = MP.attention(h, w, dict(m, mask={"size": 1}), 1e-5)
    assert np.allclose(y1[-1], (np.tile(kv[1][-1], 2) * MP.sigmoid(h[-1] @ w["g"].T)) @ w["o"].T)
    # a window of 3 against a sum written out, with the bias by distance
    y3, (k, v) = MP.attention(h, w, dict(m, mask={"size": 3}), 1e-5)
    q = (MP.rms_unit(h @ w["q"].T, 1e-5) * w["q.norm"]).reshape(6, 2, 4)
    out = np.zeros((6, 2, 6))
    for a, slope in enumerate((2.0 ** -4, 2.0 ** -8)):
        for t in range(6):
            js = [j for j in range(6) if 0 <= t - j < 3]
            e = np.array([math.exp(0.5 * (q[t, a] @ k[j]) - slope * (t - j)) for j in js])
            out[t, a] = sum(p * v[j] for p, j in zip(e / e.sum(), js))
    assert np.allclose(y3, (out.reshape(6, 12) * MP.sigmoid(h @ w["g"].T)) @ w["o"].T)


def test_the_plain_router_correction_identity_and_shared_gate():
    rng = np.random.default_rng(4)
    W, mlp = 6, _moe(5, 3, 2, 2, 1.75, shared=4)
    w = {"router": rng.normal(size=(5, W)), "correction": np.array([0.0, 0.0, 0.0, 0.0, 10.0]),
         "shared.gate": rng.normal(size=(4, W)), "shared.up": rng.normal(size=(4, W)), "shared.down": rng.normal(size=(W, 4)),
         "shared.sg": rng.normal(size=(1, W))}
    for e in range(3):
        w.update({f"e{e}.gate": rng.normal(size=(5, W)), f"e{e}.up": rng.normal(size=(5, W)), f"e{e}.down": rng.normal(size=(W, 5))})
    h = rng.normal(size=(9, W))
    chosen, weights = MP.route(h, w, mlp["router"])
    z = h @ w["router"].T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    assert (chosen[:, 0] == 4).all()                                     # the correction decides the choice ...
    assert np.allclose(weights[:, 0], 1.75 * s[:, 4])                     # ... but not the weight
    assert np.array_equal(chosen[:, 1], np.argmax(s[:, :4], axis=-1))
    got = MP.routed(h, w, mlp)
    for t in range(9):
        want = weights[t, 0] * h[t]                                       # expert 4 is the second identity expert
        e = chosen[t, 1]
        want = want + weights[t, 1] * (h[t] if e >= 3 else MP.gated_expert(h[t:t + 1], w, f"e{e}.")[0])
        want = want + MP.gated_expert(h[t:t + 1], w, "shared.")[0] * MP.sigmoid(h[t] @ w["shared.sg"][0])
        assert np.allclose(got[t], want)
    assert not np.allclose(weights.sum(-1), 1.75)                          # the weights are not rescaled to sum to one


def test_parts_declare_their_parameters_without_a_gpu():
    spec = mubasun_spec(MubasunConfig.from_dict(RAW))
    shapes = MIXERS.get("attention").param_shapes(spec.layers[0].mixer)
    assert shapes["q_norm"][0] == (32,) and shapes["k_norm"][0] == (16,) and shapes["g_proj"][0] == (48, 48)
    shared = MIXERS.get("attention")(spec.layers[2].mixer)
    assert shared.heads.n_kv_heads == 0 and shared.cache_need().window == 7 and shared.out_gate and shared.norm_whole
    ff = FEED_FORWARDS.get("routed_experts").param_shapes(spec.layers[1].feed_forward)
    assert ff["router"][0] == (7, 48) and ff["correction"][0] == (7,) and ff["shared_gate"][0] == (1, 48)
    assert FEED_FORWARDS.get("mlp").param_shapes(spec.layers[0].feed_forward)["act_params"][0] == (2,)
    with pytest.raises(ValueError):
        NORMS.get("group_rmsnorm")(PartSpec("group_rmsnorm", {"size": 48, "eps": 1e-5, "groups": 5}))
    with pytest.raises(ValueError):
        MIXERS.get("attention")(PartSpec("attention", dict(spec.layers[0].mixer.params, distance_slopes=(0.5, 0.25))))
