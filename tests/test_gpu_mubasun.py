"""Mubasun on the GPU against the plain implementation (tests/plain/mubasun_plain.py): the small kernels; the norm
over a whole projection; the router, the experts and the dense feed-forward alone; the attention mixer alone over a
cache of its own (prompts, single tokens across page and ring edges, portions, a slot handed out again, keys just
inside and just outside a window, a far key that one score singles out, a layer on another layer's keys); then whole
models through bin/trace_run under every cutting, in portions down to two tokens, through the entry point's
generation loop, and configurations drawn at random.  The configurations are small and differ from one another in
every size and constant."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import close
from plain import mubasun_plain as MP
from test_gpu_fuposun import part_step
from test_gpu_replay import Replay, run_all_cuttings

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.asarray(a)).to(DEV).to(dtype).contiguous()


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rnd(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).normal(size=shape) * scale).astype(np.float32)


def bf(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def f64(w):
    return {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


def near(got, ref, dtype, float32=1e-4):
    """How whole models are compared.  float32: by the largest difference, 1e-4 of the largest logit; a wrong mask, key,
    window, slope or expert moves these models' logits by 1e-2 and more.  bfloat16: a row is compared by the root mean
    square of its difference (mean taken off) against that of the logits, at most a tenth, and one row in thirty (or one)
    may lie beyond: the router sees the bfloat16 rounding of its input, so where two experts' scores lie within a part
    in a few hundred of each other it may choose the other one, and that row (not its neighbours) then differs by an
    expert's whole output."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if dtype == "float32":
        tol = float32 * max(1.0, float(np.abs(ref).max()))
        err = float(np.abs(got - ref).max()) if got.size else 0.0
        return err <= tol, err, tol
    if not got.size:
        return True, 0.0, 0.1
    d = got - ref
    d = d - d.mean(axis=-1, keepdims=True)
    r = ref - ref.mean(axis=-1, keepdims=True)
    e = np.sqrt((d * d).mean(axis=-1)) / np.sqrt((r * r).mean())
    over = int((e > 0.1).sum())
    allowed = max(1, len(e) // 30)
    return over <= allowed, float(np.sort(e)[-1 - min(over, allowed, len(e) - 1)]), 0.1


@pytest.fixture
def whole_model_tolerance(monkeypatch):
    import test_gpu_replay
    monkeypatch.setattr(test_gpu_replay, "close", near)


# ---- configurations -------------------------------------------------------------------------------------

def _att(heads, kv, dim, vdim, scale, window=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, identity, top, scale, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


# A: two groups in the norms; a layer without a window whose keys a windowed layer reads; a window shorter than a page;
#    key sizes above and below the value sizes; one identity expert; a reader without a feed-forward
MUBA_A = dict(architecture="Mubasun", vocab=300, width=64, max_positions=512, norm={"eps": 1e-6, "groups": 2},
              initializer_range=0.08, layers=[
                  _layer(_att(4, 2, 16, 24, 0.25), _dense(96)),
                  _layer(_att(2, 2, 24, 8, 0.2, window=9), _moe(24, 5, 1, 2, 1.7, shared=40)),
                  _layer(_att(4, 2, 16, 24, 0.25, window=33, kv_from=0), None),
                  _layer(_att(2, 2, 24, 8, 0.3, window=9, kv_from=1), _moe(16, 3, 2, 3, 0.8))])
# B: head size 64 (the tensor-core attention kernels in bfloat16), a window beyond a page, two readers on one owner with
#    a layer between, one of them with a longer window than its owner and one with none; one group (a plain RMS norm);
#    top 1; no identity experts; a routed layer without a shared expert
MUBA_B = dict(architecture="Mubasun", vocab=512, width=128, max_positions=1024, norm={"eps": 1e-5, "groups": 1},
              initializer_range=0.06, layers=[
                  _layer(_att(4, 1, 64, 64, 0.125, window=70), _moe(64, 6, 0, 1, 1.0, shared=96)),
                  _layer(_att(2, 2, 64, 32, 0.11), _dense(192)),
                  _layer(_att(4, 1, 64, 64, 0.1, window=130, kv_from=0), _moe(32, 4, 0, 2, 2.0)),
                  _layer(_att(2, 2, 64, 32, 0.11, window=64, kv_from=1), None),
                  _layer(_att(4, 1, 64, 64, 0.125, kv_from=0), _dense(64))])
# C: a width, head sizes and a vocabulary that are no multiple of 8, five groups, a window of one token, one head
#    everywhere in one layer, more identity experts than experts, every expert chosen
MUBA_C = dict(architecture="Mubasun", vocab=301, width=100, max_positions=400, norm={"eps": 1e-4, "groups": 5},
              initializer_range=0.07, layers=[
                  _layer(_att(5, 5, 12, 20, 0.3), _dense(70)),
                  _layer(_att(3, 1, 20, 12, 0.22, window=1), _moe(36, 2, 3, 2, 3.0, shared=20)),
                  _layer(_att(1, 1, 8, 8, 0.35, window=11), None),
                  _layer(_att(3, 3, 4, 28, 0.4, window=65), _moe(12, 3, 1, 4, 0.5))])
CONFIGS = {"A": (MUBA_A, 3), "B": (MUBA_B, 4), "C": (MUBA_C, 5)}
LENGTHS = [70, 33, 129, 45, 100, 64]
LENGTHS_B = [170, 33, 257, 45, 100, 64]


def make_folder(base, name, storage, peaky):
    """Random weights.  The corrections are a fifth of what the norm weights' spread would make them, so that scores and
    corrections both decide the choice; ``peaky`` scales what decides where attention looks (the weights of the query and
    key norms, which set the size of queries and keys after their norm) and the router's matrix."""
    from quicknn_b200.config import MUBASUN, MubasunConfig
    from quicknn_b200.weights import random_tensors, write_safetensors
    raw, seed = CONFIGS[name]
    cfg = MubasunConfig.from_dict(raw)
    d = os.path.join(str(base), f"muba{name}_{storage}{'_peaky' if peaky else ''}")
    os.makedirs(d, exist_ok=True)
    tensors = dict(random_tensors(MUBASUN, cfg, seed, torch.float32, 0.2))
    for k in list(tensors):
        if k.endswith("mlp.correction"):
            tensors[k] = tensors[k] * 0.2
        elif k.endswith("mlp.act"):
            tensors[k] = tensors[k] * 4.0                       # softplus(p), softplus(q) well away from log 2
        elif peaky and k.endswith(("q.norm", "k.norm")):
            tensors[k] = tensors[k] * 2.5
        elif peaky and k.endswith("mlp.router"):
            tensors[k] = tensors[k] * 4.0
    dt = torch.float32 if storage == "float32" else torch.bfloat16
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.to(dt) for k, v in tensors.items()})
    return d


@pytest.fixture(scope="module")
def muba(tmp_path_factory):
    base = tmp_path_factory.mktemp("mubasun")
    made = {}

    def get(name, storage="float32", peaky=False):
        key = (name, storage, peaky)
        if key not in made:
            folder = make_folder(base, name, storage, peaky)
            made[key] = (folder, MP.PlainMubasun(folder))
        return made[key]
    return get


def prompts(name, lengths, seed=0):
    rng = np.random.default_rng(100 + seed)
    return [rng.integers(1, CONFIGS[name][0]["vocab"], n).tolist() for n in lengths]


# ---- the small kernels ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_in_groups_alone_after_an_add_and_with_the_embedding(dtype):
    from quicknn_b200.kernels import ops
    tol = 2e-5 if dtype == torch.float32 else 0.02
    for rows, width, groups in ((3, 100, 5), (70, 64, 2), (5, 2304, 1), (2, 12288, 4), (9, 48, 48), (4, 36, 3)):
        x, w = bf(rnd((rows, width), 1, 2.0) + 0.7), bf(rnd(width, 3, 0.2) + 1.0)
        ref = MP.group_norm(x.astype(np.float64), w.astype(np.float64), groups, 1e-5)
        assert np.abs(host(ops.group_rmsnorm(dev(x, dtype), dev(w, dtype), 1e-5, groups, dtype)) - ref).max() < tol * np.abs(ref).max()
        assert np.abs(host(ops.group_rmsnorm(dev(x), dev(w, dtype), 1e-5, groups, dtype)) - ref).max() < tol * np.abs(ref).max()
        # the stream takes both sublayers' outputs; the next layer's norm comes out of the same kernel
        resid, a, b = rnd((rows, width), 4, 3.0), bf(rnd((rows, width), 5)), bf(rnd((rows, width), 6, 2.0))
        for first, second in ((a, b), (a, None), (None, b)):
            r = dev(resid)
            normed = ops.add2_group_rmsnorm(r, None if first is None else dev(first, dtype),
                                            None if second is None else dev(second, dtype), dev(w, dtype), 1e-5, groups, dtype)
            want = resid.astype(np.float64) + (0 if first is None else first) + (0 if second is None else second)
            assert np.abs(host(r) - want).max() < 3e-6 * np.abs(want).max()                  # the stream itself is float32
            ref = MP.group_norm(want, w.astype(np.float64), groups, 1e-5)
            assert np.abs(host(normed) - ref).max() < tol * np.abs(ref).max()
        r = dev(resid)
        assert ops.add2_group_rmsnorm(r, dev(a, dtype), dev(b)) is None                      # the last layer: no norm follows
        assert np.abs(host(r) - (resid.astype(np.float64) + a + b)).max() < 3e-6 * np.abs(resid).max()
    # embedded rows plus the vectors of their positions, and the first norm
    V, P, width, groups = 50, 40, 72, 3
    table, pos_table, w = bf(rnd((V, width), 7)), bf(rnd((P, width), 8)), bf(rnd(width, 9, 0.2) + 1.0)
    tokens, positions = np.array([0, 49, 7, 7, 3], dtype=np.int32), np.array([0, 1, 39, 0, 20], dtype=np.int32)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)  # noqa: E731
    want = table[tokens].astype(np.float64) * 1.5 + pos_table[positions]
    x, normed = ops.embed_pos(i32(tokens), dev(table, dtype), 1.5, dev(pos_table, dtype), i32(positions), dev(w, dtype), 1e-5,
                              groups, dtype)
    assert x.dtype == torch.float32 and np.abs(host(x) - want).max() < 1e-6 * np.abs(want).max()
    ref = MP.group_norm(want, w.astype(np.float64), groups, 1e-5)
    assert np.abs(host(normed) - ref).max() < tol * np.abs(ref).max()
    x2, none = ops.embed_pos(i32(tokens), dev(table, dtype), 1.5, dev(pos_table, dtype), i32(positions))
    assert none is None and torch.equal(x2, x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_xielu_and_the_gate_per_element(dtype):
    from quicknn_b200.kernels import ops
    tol = 1e-6 if dtype == torch.float32 else 0.01
    z = bf(np.concatenate([rnd(500, 1, 3.0), [-40.0, -1e-3, 0.0, 1e-3, 12.0]]).astype(np.float32)).reshape(5, 101)
    for p, q in ((0.3, -0.7), (-5.0, 4.0), (0.0, 0.0)):
        ap, an = float(MP.softplus(np.float64(p))), 0.5 + float(MP.softplus(np.float64(q)))
        got = host(ops.xielu_(dev(z, dtype), ap, an))
        want = MP.xielu(z.astype(np.float64), p, q)
        assert np.abs(got - want).max() < tol * np.abs(want).max()
    o, g = bf(rnd((7, 40), 2)), bf(rnd((7, 100), 3, 3.0))
    for col0 in (0, 60, 13):
        t = dev(o, dtype)
        ops.sigmoid_gate_(t, dev(g, dtype), col0)
        want = o.astype(np.float64) * MP.sigmoid(g[:, col0:col0 + 40].astype(np.float64))
        assert np.abs(host(t) - want).max() < tol * 4 * np.abs(want).max()
    t = dev(o, dtype)
    ops.sigmoid_gate_(t, dev(g[:, :40]))                                   # float32 logits beside rows of either type
    assert np.abs(host(t) - o * MP.sigmoid(g[:, :40].astype(np.float64))).max() < tol * 4 * np.abs(o).max()


@pytest.mark.parametrize("hd,norm_dim,nq,nk", [(16, 16, 3, 2), (24, 20, 4, 1), (8, 8, 1, 1), (64, 64, 4, 1), (128, 128, 2, 2),
                                               (32, 12, 5, 5), (256, 256, 1, 1)])
@pytest.mark.parametrize("c_in,spare", [(3, 5), (8, 16)])
def test_one_norm_over_all_heads_of_a_projection(hd, norm_dim, nq, nk, c_in, spare):
    """Queries and keys each pass one RMS norm over all their heads at once (the columns that a head carries beyond its
    size do not count), with a weight per head and column; values pass untouched."""
    from quicknn_b200.kernels import ops
    T, eps = 7, 1e-5
    nv = nk * hd
    width = (nq + nk) * hd + nv
    x = bf(rnd((T, width + spare), 1))
    for n, c0 in ((nq, c_in), (nk, c_in + nq * hd)):                          # what a head carries beyond its size is zero
        x[:, c0:c0 + n * hd].reshape(T, n, hd)[..., norm_dim:] = 0.0
    wq, wk = bf(rnd(nq * norm_dim, 3, 0.2) + 1), bf(rnd(nk * norm_dim, 4, 0.2) + 1)

    def plain_heads(c0, n, w):
        h = x[:, c0:c0 + n * hd].astype(np.float64).reshape(T, n, hd)
        flat = h[..., :norm_dim].reshape(T, n * norm_dim)
        h[..., :norm_dim] = (MP.rms_unit(flat, eps) * w).reshape(T, n, norm_dim)
        return h.reshape(T, n * hd)
    want = np.concatenate([plain_heads(c_in, nq, wq), plain_heads(c_in + nq * hd, nk, wk),
                           x[:, c_in + (nq + nk) * hd:c_in + width].astype(np.float64)], axis=1)
    for dtype in (torch.float32, torch.bfloat16):
        src = dev(x, dtype)
        ops.head_prep(src, c_in, nq, nk, nv, hd, q_norm=dev(wq, dtype), k_norm=dev(wk, dtype), norm_dim=norm_dim, eps=eps,
                      rot_dim=0, norm_whole=True)
        got = host(src)
        assert np.abs(got[:, c_in:c_in + width] - want).max() < (3e-5 if dtype == torch.float32 else 0.02) * np.abs(want).max()
        assert np.array_equal(got[:, :c_in], x[:, :c_in].astype(np.float64))
        assert np.array_equal(got[:, c_in + width:], x[:, c_in + width:].astype(np.float64))
        q_only = dev(x[:, c_in:c_in + nq * hd].copy(), dtype)               # a layer on another layer's keys: queries alone
        ops.head_prep(q_only, 0, nq, 0, 0, hd, q_norm=dev(wq, dtype), norm_dim=norm_dim, eps=eps, rot_dim=0, norm_whole=True)
        assert np.abs(host(q_only) - want[:, :nq * hd]).max() < (3e-5 if dtype == torch.float32 else 0.02) * np.abs(want).max()


# ---- the feed-forwards alone ---------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,ff,rows", [(48, 72, 5), (100, 36, 130), (256, 512, 300)])
def test_dense_feed_forward_with_its_two_learned_numbers(dtype, W, ff, rows):
    from quicknn_b200.parts import FEED_FORWARDS, PartSpec
    spec = PartSpec("mlp", {"hidden_size": W, "intermediate_size": ff, "activation": "xielu"})
    part = FEED_FORWARDS.get("mlp")(spec)
    w = {"up": bf(rnd((ff, W), 1, 0.3)), "down": bf(rnd((W, ff), 2, 0.3)), "act": np.array([1.3, -2.1], dtype=np.float32)}
    part.load({"up_proj": dev(w["up"], dtype), "down_proj": dev(w["down"], dtype), "act_params": dev(w["act"], dtype)}, dtype, DEV)
    x = bf(rnd((rows, W), 3))
    want = MP.dense(x.astype(np.float64), f64(dict(w, act=bf(w["act"]) if dtype == torch.bfloat16 else w["act"])))
    got = host(part.forward(dev(x, dtype), None))
    assert np.abs(got - want).max() < (3e-5 if dtype == torch.float32 else 0.03) * np.abs(want).max()


def _routed_part(W, mlp, dtype, seed, router_scale=3.0, correction=None):
    from quicknn_b200.parts import FEED_FORWARDS, PartSpec
    r = mlp["router"]
    E, n_id = r["experts"], r["identity"]
    shared = None
    if mlp.get("shared"):
        shared = PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": mlp["shared"]["ff"], "activation": "silu"})
    spec = PartSpec("routed_experts", {
        "hidden_size": W, "intermediate_size": mlp["expert"]["ff"], "experts": E, "top": r["top"], "activation": "silu",
        "score": "softmax", "renormalize": False, "weight_on": "output", "correction": True, "identity": n_id,
        "route_scale": r["scale"], "shared": shared, "shared_gate": shared is not None})
    part = FEED_FORWARDS.get("routed_experts")(spec)
    ff = mlp["expert"]["ff"]
    w = {"router": rnd((E + n_id, W), seed, router_scale / W ** 0.5),
         "correction": rnd(E + n_id, seed + 1, 0.05) if correction is None else np.asarray(correction, dtype=np.float32)}
    names = {"router": "router", "correction": "correction"}
    for e in range(E):
        for j, n in enumerate(("gate", "up", "down")):
            w[f"e{e}.{n}"] = rnd((W, ff) if n == "down" else (ff, W), seed + 10 * e + j + 2, 0.3)
            names[f"e{e}.{n}"] = f"experts.{e}.{n}_proj"
    if shared is not None:
        sf = mlp["shared"]["ff"]
        w.update({"shared.gate": rnd((sf, W), seed + 500, 0.3), "shared.up": rnd((sf, W), seed + 501, 0.3),
                  "shared.down": rnd((W, sf), seed + 502, 0.3), "shared.sg": rnd((1, W), seed + 503, 0.5)})
        names.update({"shared.gate": "shared.gate_proj", "shared.up": "shared.up_proj", "shared.down": "shared.down_proj",
                      "shared.sg": "shared_gate"})
    w = {k: bf(v) for k, v in w.items()}
    part.load({names[k]: dev(v, torch.float32 if k == "correction" else dtype) for k, v in w.items()}, dtype, DEV)
    return part, f64(w)


def _clear_choices(x, w, r, margin):
    """Rows whose choice does not hang on less than ``margin`` between the last chosen and the first left-out expert."""
    z = x @ w["router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    c = np.sort(s / s.sum(-1, keepdims=True) + w["correction"], axis=-1)[:, ::-1]
    top = int(r["top"])
    return np.ones(len(x), dtype=bool) if top >= c.shape[1] else (c[:, top - 1] - c[:, top]) > margin


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,mlp,rows", [
    (48, _moe(24, 5, 1, 2, 1.7, shared=40), 70), (64, _moe(16, 3, 2, 3, 0.8), 33), (100, _moe(36, 2, 3, 2, 3.0, shared=20), 9),
    (128, _moe(64, 6, 0, 1, 1.0, shared=96), 300), (40, _moe(12, 3, 1, 4, 0.5), 17), (64, _moe(32, 16, 2, 4, 2.5, shared=8), 1),
    (256, _moe(128, 8, 1, 2, 1.0, shared=64), 700)])
def test_routed_experts_with_identity_experts_and_a_gated_shared_expert(dtype, W, mlp, rows):
    part, w = _routed_part(W, mlp, dtype, 40)
    x = bf(rnd((rows, W), 5))
    want = MP.routed(x.astype(np.float64), w, mlp)
    got = host(part.forward(dev(x, dtype), None))
    clear = _clear_choices(x.astype(np.float64), w, mlp["router"], 1e-6 if dtype == torch.float32 else 3e-3)
    assert clear.mean() > 0.7
    tol = (3e-5 if dtype == torch.float32 else 0.03) * np.abs(want).max()
    assert np.abs(got - want)[clear].max() < tol


def test_the_router_ranks_by_corrected_scores_and_weighs_by_the_scores():
    """A correction lifts one expert and one identity expert above all others: they are chosen for every row, weighted by
    their own small scores times the scale; among equal choice scores the lower index wins."""
    from quicknn_b200.kernels import ops
    W, E, n_id, top = 32, 4, 2, 3
    router, x = bf(rnd((E + n_id, W), 1, 0.4)), bf(rnd((50, W), 2))
    corr = np.array([0.0, 0.0, 5.0, 0.0, 0.0, 7.0], dtype=np.float32)
    for dtype in (torch.float32, torch.bfloat16):
        sel_e, sel_w = ops.moe_route(dev(x, dtype), dev(router, dtype), top, "softmax", False, dev(corr), 2.5)
        chosen, weights = MP.route(x.astype(np.float64), {"router": router.astype(np.float64), "correction": corr.astype(np.float64)},
                                   {"top": top, "scale": 2.5})
        e, wt = sel_e.cpu().numpy().reshape(50, top), host(sel_w).reshape(50, top)
        assert (e[:, 0] == 5).all() and (e[:, 1] == 2).all()
        order = np.argsort(e, axis=-1), np.argsort(chosen, axis=-1)
        same = (np.take_along_axis(e, order[0], -1) == np.take_along_axis(chosen, order[1], -1)).all(-1)
        assert same.mean() > (0.99 if dtype == torch.float32 else 0.9)
        got, ref = np.take_along_axis(wt, order[0], -1)[same], np.take_along_axis(weights, order[1], -1)[same]
        assert np.abs(got - ref).max() < (1e-5 if dtype == torch.float32 else 0.02) * ref.max()
    # ties: all logits equal, so every score is 1 / (E + n_id) and the first ``top`` indices are chosen
    sel_e, sel_w = ops.moe_route(torch.zeros((3, W), device=DEV), dev(router), top, "softmax", False, torch.zeros(E + n_id, device=DEV), 1.0)
    assert sel_e.cpu().numpy().reshape(3, top).tolist() == [[0, 1, 2]] * 3 and np.allclose(host(sel_w), 1.0 / (E + n_id))
