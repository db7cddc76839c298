"""Gunirax without a GPU: the configuration (registry, round trip, rules reported by name), its layout (parts, tensor
names, the schedule of a looped stack), a random folder that the plain implementation reads, and the plain mechanisms
against hand-made cases."""
import copy
import json
import os

import numpy as np
import pytest
import torch

from plain import gunirax_plain as GP


def _left(heads=4, kv=2, dim=8, scale=0.3, chunk=5, dims=4, scaling=True):
    rot = {"base": 1000.0, "dims": dims}
    if scaling:
        rot["scaling"] = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def _right(heads=2, dim=4, vdim=6, decay=(0.5, 0.97)):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _moe(ff=12, experts=6, top=2, scale=1.5, count=3, keep=2, shared=10):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


RAW = dict(architecture="Gunirax", vocab=90, width=24, embedding={"scale": 2.0}, norm={"eps": 1e-5},
           loop={"start": 1, "stop": 3, "times": 3}, initializer_range=0.08, layers=[
               {"type": "hgrn2", "mixer": {"heads": 2, "dim": 4, "vdim": 8}, "mlp": {"kind": "dense", "ff": 40}},
               {"type": "parallel", "mixer": {"left": _left(), "right": _right()}, "mlp": _moe()},
               {"type": "parallel", "mixer": {"left": _left(2, 1, 12, 0.2, None, 12, False), "right": _right(1, 8, 4, (0.9,))},
                "mlp": None},
               {"type": "hgrn2", "mixer": {"heads": 1, "dim": 6, "vdim": 4}, "mlp": _moe(8, 4, 1, 0.7, 1, 1, None)}])


def test_registry_round_trip_and_the_schedule_of_a_looped_stack():
    from quicknn_b200.config import GUNIRAX, GuniraxConfig, find_architecture
    assert find_architecture({"architecture": "Gunirax"}) is GUNIRAX
    cfg = GuniraxConfig.from_dict(RAW)
    assert GuniraxConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.layer_runs() == ((0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False))
    assert [(r["layer"], r["restart"]) for r in GP.layer_runs(RAW)] == list(cfg.layer_runs())
    spec = GUNIRAX.build_spec(cfg)
    assert [(e.layer, e.cache, e.add_embedding) for e in spec.schedule] == [
        (0, 0, False), (1, 1, False), (2, 2, False), (1, 3, True), (2, 4, False), (1, 5, True), (2, 6, False), (3, 7, False)]
    assert spec.n_cache_lines() == 8 and all(e.writes_cache for e in spec.schedule)
    # no loop at all, and a loop over everything
    plain = GuniraxConfig.from_dict({k: v for k, v in RAW.items() if k != "loop"})
    assert plain.layer_runs() == tuple((i, False) for i in range(4))
    every = GuniraxConfig.from_dict(dict(RAW, loop={"start": 0, "stop": 4, "times": 2}))
    assert every.layer_runs() == tuple((i, False) for i in range(4)) + ((0, True), (1, False), (2, False), (3, False))


def test_layout_parts_and_tensor_names():
    from quicknn_b200.config import GUNIRAX, GuniraxConfig
    from quicknn_b200.parts import expected_tensors
    spec = GUNIRAX.build_spec(GuniraxConfig.from_dict(RAW))
    assert [l.mixer.kind for l in spec.layers] == ["hgrn2", "parallel", "parallel", "hgrn2"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == \
        ["gated_mlp", "routed_experts", None, "routed_experts"]
    left = spec.layers[1].mixer.params["branches"]["left"]
    assert left.kind == "sigmoid_attention" and left.params["mask"] == {"kind": "chunk", "size": 5}
    assert spec.layers[2].mixer.params["branches"]["left"].params["mask"]["kind"] == "causal"
    assert spec.layers[1].feed_forward.params["groups"] == (3, 2) and not spec.layers[1].feed_forward.params["gated"]
    names = expected_tensors(spec)
    for n, shape in {"embed": (90, 24), "head": (90, 24), "final.norm": (24,), "final.norm.alpha": (), "final.norm.b": (24,),
                     "l0.norm1.alpha": (), "l0.mix.f.b": (8,), "l0.mix.lower": (8,), "l0.mix.norm": (8,), "l0.mix.o": (24, 16),
                     "l0.mlp.gate": (40, 24), "l1.mix.left.q": (32, 24), "l1.mix.left.k.b": (16,), "l1.mix.left.talk": (4, 4),
                     "l1.mix.left.pb": (4,), "l1.mix.left.g": (4, 24), "l1.mix.left.out": (24,), "l1.mix.right.norm": (12,),
                     "l1.mix.right.g": (12, 24), "l1.mlp.e5.up": (12, 24), "l1.mlp.e0.down": (24, 12), "l1.mlp.correction": (6,),
                     "l1.mlp.shared.up": (10, 24), "l3.mlp.router": (4, 24)}.items():
        assert names[n][0] == shape, n
    assert "l1.mix.left.v" not in names and "l2.norm2" not in names and "l3.mlp.shared.up" not in names
    assert "l2.norm2" in spec.optional_tensors


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][1]["mixer"]["left"].update(vdim=9), "vdim must equal dim"),
    (lambda r: r["layers"][1]["mixer"]["left"].update(kv_heads=3), "do not divide"),
    (lambda r: r["layers"][1]["mixer"]["left"]["mask"].update(size=0), "mask.size"),
    (lambda r: r["layers"][1]["mixer"]["left"]["rot"].update(dims=5), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(decay=[0.5]), "one number per head"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(decay=[0.5, 1.5]), "lies in [0, 1]"),
    (lambda r: r["layers"][0]["mixer"].update(dim=300), "at most 256"),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=6), "cannot give"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda r: r["loop"].update(stop=5), "loop"),
    (lambda r: r["loop"].update(times=0), "loop"),
    (lambda r: r["norm"].update(eps=0.0), "norm.eps"),
])
def test_every_broken_rule_is_named(change, word):
    from quicknn_b200.config import ConfigError, GuniraxConfig
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError) as e:
        GuniraxConfig.from_dict(raw)
    assert word in str(e.value)


def test_a_layer_type_or_feed_forward_kind_that_does_not_exist():
    from quicknn_b200.config import ConfigError, GuniraxConfig
    for change in (lambda r: r["layers"][0].update(type="attention"), lambda r: r["layers"][0]["mlp"].update(kind="glu")):
        raw = copy.deepcopy(RAW)
        change(raw)
        with pytest.raises(ConfigError):
            GuniraxConfig.from_dict(raw)


def test_a_random_folder_loads_and_the_plain_model_reads_it(tmp_path):
    from quicknn_b200.config import GUNIRAX, GuniraxConfig, load_config
    from quicknn_b200.weights import write_model_folder
    cfg = GuniraxConfig.from_dict(RAW)
    folder = write_model_folder(str(tmp_path / "m"), GUNIRAX, cfg, seed=5)
    arch, again = load_config(folder)
    assert arch is GUNIRAX and again == cfg
    plain = GP.PlainGunirax(folder)
    logits, streams = GP.forward(plain.cfg, plain.w, [3, 1, 4, 1, 5, 9, 2, 6], return_layers=True)
    assert logits.shape == (8, 90) and streams.shape == (8, 8, 24) and np.isfinite(logits).all()


def test_rotary_frequencies_of_the_library_are_the_plain_ones():
    from quicknn_b200.config.tumudra import RotaryConfig
    from quicknn_b200.parts import POSITIONS
    for rot in ({"base": 20000.0, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}},
                {"base": 100.0, "dims": 6}, {"base": 1e6, "dims": 64, "scaling": {"factor": 32.0, "low": 2.0, "high": 3.0,
                                                                                  "original": 8192}}):
        part = RotaryConfig.parse(rot, "rot").part(64, "interleaved")
        got = POSITIONS.get(part.kind)(part).frequencies().numpy()
        assert np.allclose(got, GP.rotary_frequencies(rot), rtol=1e-12, atol=0)
    # the three regimes are all met by the first case: kept, divided, blended
    f0 = 20000.0 ** (-2.0 * np.arange(16) / 32)
    f = GP.rotary_frequencies({"base": 20000.0, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}})
    ratio = f / f0
    assert (ratio == 1.0).any() and np.isclose(ratio, 0.25).any() and ((ratio > 0.26) & (ratio < 0.99)).any()


def test_chunks_count_from_the_start_of_the_sequence():
    see = GP.chunk_visible(7, 3)
    assert see.astype(int).tolist() == [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0],
                                        [0, 0, 0, 1, 0, 0, 0], [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0],
                                        [0, 0, 0, 0, 0, 0, 1]]
    assert GP.chunk_visible(4, 1).astype(int).tolist() == np.eye(4, dtype=int).tolist()
    # the same positions, cut out of a longer sequence
    assert (GP.chunk_visible(5, 4, first_position=6) == GP.chunk_visible(11, 4)[6:, 6:]).all()


def test_sigmoid_attention_by_hand():
    """One head, no rotation: the output is the gate times the sum over the chunk's keys of sigmoid(score + pb) k_j."""
    rng = np.random.default_rng(0)
    n, W, D = 5, 6, 4
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": 0.7, "rot": {"base": 10.0, "dims": 0}, "mask": {"size": 2}}
    w = {"q": rng.normal(size=(D, W)), "q.b": rng.normal(size=D), "k": rng.normal(size=(D, W)), "k.b": rng.normal(size=D),
         "talk": np.array([[1.3]]), "pb": np.array([-0.4]), "g": rng.normal(size=(1, W)), "o": np.eye(D)}
    h = rng.normal(size=(n, W))
    got = GP.sigmoid_attention(h, w, "", m, 1e-6)
    q = h @ w["q"].T + w["q.b"]
    k = h @ w["k"].T + w["k.b"]
    unit = lambda a: a / np.sqrt((a * a).mean(-1, keepdims=True) + 1e-6)  # noqa: E731
    for i in range(n):
        want = np.zeros(D)
        for j in range((i // 2) * 2, i + 1):
            want += 1.3 * GP.sigmoid(0.7 * unit(q[i]) @ unit(k[j]) - 0.4) * k[j]
        want *= GP.sigmoid(h[i] @ w["g"][0])
        assert np.allclose(got[i], want)


def test_the_memories_as_sums_over_earlier_tokens():
    rng = np.random.default_rng(1)
    n, W = 6, 5
    h = rng.normal(size=(n, W))
    m = {"heads": 1, "dim": 3, "vdim": 2, "decay": [0.8]}
    w = {k: rng.normal(size=s) for k, s in {"q": (3, W), "k": (3, W), "v": (2, W), "g": (2, W), "o": (W, 2)}.items()}
    w["norm"] = np.ones(2)
    got = GP.lightning(h, w, "", m, 1e-6)
    q, k, v = GP.silu(h @ w["q"].T), GP.silu(h @ w["k"].T), GP.silu(h @ w["v"].T)
    o = np.stack([sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(n)])
    assert np.allclose(got, (GP.rms_unit(o, 1e-6) * GP.sigmoid(h @ w["g"].T)) @ w["o"].T)
    # hgrn2: the key is what the forget gate lets go; a lower bound of 1 freezes the (empty) state
    w2 = {"q": rng.normal(size=(3, W)), "f": rng.normal(size=(3, W)), "f.b": rng.normal(size=3), "lower": np.array([0.0, 0.5, 0.9]),
          "v": rng.normal(size=(2, W)), "norm": np.array([1.0, 2.0]), "o": np.eye(2)}
    got = GP.hgrn2(h, w2, "", {"heads": 1, "dim": 3, "vdim": 2}, 1e-6)
    f = w2["lower"] + (1 - w2["lower"]) * GP.sigmoid(h @ w2["f"].T + w2["f.b"])
    q = GP.silu(h @ w2["q"].T)
    o = np.zeros((n, 2))
    for t in range(n):
        for j in range(t + 1):
            keep = np.prod(f[j + 1:t + 1], axis=0)
            o[t] += ((1 - f[j]) * keep * q[t]).sum() * (h[j] @ w2["v"].T)
    assert np.allclose(got, GP.rms_unit(o, 1e-6) * w2["norm"])
    frozen = GP.hgrn2(h, dict(w2, lower=np.ones(3)), "", {"heads": 1, "dim": 3, "vdim": 2}, 1e-6)
    assert np.abs(frozen).max() == 0.0


def test_the_choice_stays_within_the_best_groups_and_weights_ignore_the_correction():
    W = 4
    h = np.eye(W)[:1] * 1.0                                  # one token; the router's first column gives the logits
    logits = np.array([2.0, -3.0, 1.5, 1.4, 0.0, 0.1, -1.0, 3.0])
    w = {"router": np.zeros((8, W)), "correction": np.array([0.0, 0.0, 0.0, 0.0, 0.4, 0.4, 0.0, -0.5])}
    w["router"][:, 0] = logits
    r = {"experts": 8, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    s = GP.sigmoid(logits)
    c = s + w["correction"]
    groups = [c[0] + c[1], c[2] + c[3], c[4] + c[5], c[6] + c[7]]
    assert np.argsort(groups)[::-1][:2].tolist() == [2, 1]       # experts 4, 5 (lifted by the correction) and 2, 3
    chosen, weights = GP.route(h, w, "", r)
    assert sorted(chosen[0].tolist()) == [2, 4, 5]               # expert 0 and 7 score higher but their groups are out
    assert np.allclose(weights[0], s[chosen[0]] / s[chosen[0]].sum() * 2.0)
    # negative ranking values: what lies outside the kept groups never wins against them
    w["correction"] = np.full(8, -5.0)
    w["correction"][6:] = -4.0
    chosen, _ = GP.route(h, w, "", dict(r, groups={"count": 4, "keep": 1}, top=2))
    assert sorted(chosen[0].tolist()) == [6, 7]
    # one group: a plain choice of the best
    chosen, _ = GP.route(h, dict(w, correction=np.zeros(8)), "", dict(r, groups={"count": 1, "keep": 1}))
    assert sorted(chosen[0].tolist()) == [0, 2, 7]


def test_dynamic_tanh_and_the_feed_forwards():
    x = np.array([[0.0, 1.0, -2.0]])
    w = {"n": np.array([1.0, 2.0, 3.0]), "n.b": np.array([0.5, 0.0, -1.0]), "n.alpha": np.array(0.5)}
    assert np.allclose(GP.dynamic_tanh(x, w, "n"), [[0.5, 2 * np.tanh(0.5), 3 * np.tanh(-1.0) - 1.0]])
    e = {"up": np.array([[1.0, 0.0], [-1.0, 0.0]]), "down": np.array([[1.0, 1.0]])}
    assert np.allclose(GP.relu2_expert(np.array([[3.0, 7.0]]), e, ""), [[9.0]])
    assert np.allclose(GP.relu2_expert(np.array([[-2.0, 7.0]]), e, ""), [[4.0]])
