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
                  _layer(_att(4, 1, 64, 64, 0.14, window=70), _moe(64, 6, 0, 1, 1.0, shared=96)),
                  _layer(_att(2, 2, 64, 32, 0.11), _dense(192)),
                  _layer(_att(4, 1, 64, 64, 0.1, window=130, kv_from=0), _moe(32, 4, 0, 2, 2.0)),
                  _layer(_att(2, 2, 64, 32, 0.11, window=64, kv_from=1), None),
                  _layer(_att(4, 1, 64, 64, 0.14, kv_from=0), _dense(64))])
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
    o, g = bf(rnd((7, 40), 2)), bf(rnd((7, 104), 3, 3.0))
    for col0 in (0, 64, 13, 60):              # whole 16-byte pieces (eight columns at a time), and not
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
    (128, _moe(64, 6, 0, 1, 1.0, shared=96), 300), (40, _moe(12, 3, 1, 4, 0.5), 17), (64, _moe(32, 16, 3, 4, 2.2, shared=8), 1),
    (256, _moe(128, 8, 1, 2, 1.0, shared=64), 700), (96, _moe(8, 40, 3, 6, 1.2, shared=16), 150),
    (64, _moe(16, 70, 0, 16, 0.7), 40)])
def test_routed_experts_with_identity_experts_and_a_gated_shared_expert(dtype, W, mlp, rows):
    part, w = _routed_part(W, mlp, dtype, 40)
    x = bf(rnd((rows, W), 5))
    want = MP.routed(x.astype(np.float64), w, mlp)
    got = host(part.forward(dev(x, dtype), None))
    n_out = mlp["router"]["experts"] + mlp["router"]["identity"]          # scores are about 1 / n_out: so is a margin
    clear = _clear_choices(x.astype(np.float64), w, mlp["router"], (1e-6 if dtype == torch.float32 else 3e-3) * 8 / max(8, n_out))
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
        sel_e, sel_w = ops.moe_route(dev(x, dtype), dev(router, dtype), top, "softmax", False, dev(corr), 2.25)
        chosen, weights = MP.route(x.astype(np.float64), {"router": router.astype(np.float64), "correction": corr.astype(np.float64)},
                                   {"top": top, "scale": 2.25})
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


def test_rows_behind_the_routers_give_their_logits_and_take_no_part_in_the_choice():
    """The shared expert's gate rides in the router's kernel as one more row of its matrix."""
    from quicknn_b200.kernels import ops
    for W, E, top, extra in ((40, 5, 2, 1), (100, 3, 3, 2), (64, 33, 4, 1)):
        w, x = bf(rnd((E + extra, W), 11, 0.5)), bf(rnd((37, W), 12))
        corr = rnd(E, 13, 0.05)
        for dtype in (torch.float32, torch.bfloat16):
            e0, w0 = ops.moe_route(dev(x, dtype), dev(w[:E], dtype), top, "softmax", False, dev(corr), 1.3)
            e1, w1, more = ops.moe_route(dev(x, dtype), dev(w, dtype), top, "softmax", False, dev(corr), 1.3, extra=extra)
            assert torch.equal(e0, e1) and torch.equal(w0, w1)
            want = x.astype(np.float64) @ w[E:].astype(np.float64).T
            assert more.shape == (37, extra) and np.abs(host(more) - want).max() < 1e-5 * max(1.0, np.abs(want).max())


def test_an_identity_expert_returns_the_row_itself():
    """The corrections put every row on the two identity experts: the output is the row times the sum of their two
    scores times the scale, and no expert's matrices take part (they hold NaN)."""
    W, mlp = 48, _moe(16, 3, 2, 2, 1.5)
    for dtype in (torch.float32, torch.bfloat16):
        part, w = _routed_part(W, mlp, dtype, 60, correction=[0.0, 0.0, 0.0, 9.0, 8.0])
        part.w_gate_up.fill_(float("nan"))
        part.w_down.fill_(float("nan"))
        for rows in (1, 9, 300):
            x = bf(rnd((rows, W), 6))
            z = x.astype(np.float64) @ w["router"].T
            s = np.exp(z - z.max(-1, keepdims=True))
            s = s / s.sum(-1, keepdims=True)
            want = x * (1.5 * (s[:, 3] + s[:, 4]))[:, None]
            got = host(part.forward(dev(x, dtype), None))
            assert np.abs(got - want).max() < (3e-5 if dtype == torch.float32 else 0.02) * np.abs(want).max()


# ---- the attention mixer alone ---------------------------------------------------------------------------------

def _attention_mixer(W, m, dtype, seed, shared=False, tie_qk=False, eps=1e-5):
    from quicknn_b200.config.mubasun import distance_slopes
    from quicknn_b200.parts import MIXERS, PartSpec
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = (m.get("mask") or {}).get("size")
    spec = PartSpec("attention", {"hidden_size": W, "n_heads": H, "n_kv_heads": G, "head_dim": d, "v_head_dim": dv,
                                  "scale": m["scale"], "softcap": None, "window": size, "bias": False,
                                  "qk_norm": {"eps": eps, "over": "projection"}, "distance_slopes": distance_slopes(H),
                                  "out_gate": True, "shared_kv": shared, "position": PartSpec("none", {"head_dim": d})})
    mixer = MIXERS.get("attention")(spec)
    w = {"q": rnd((H * d, W), seed + 1, 0.3), "k": rnd((G * d, W), seed + 2, 0.3), "v": rnd((G * dv, W), seed + 3, 0.3),
         "o": rnd((W, H * dv), seed + 4, 0.3), "g": rnd((H * dv, W), seed + 5, 0.3),
         "q.norm": rnd(H * d, seed + 6, 0.2) + 1, "k.norm": rnd(G * d, seed + 7, 0.2) + 1}
    if tie_qk:                        # a row's key points where its query points, in every head
        w["q"] = np.concatenate([w["k"][(h // (H // G)) * d:(h // (H // G) + 1) * d] for h in range(H)])
        w["q.norm"], w["k.norm"] = np.ones(H * d, dtype=np.float32), np.ones(G * d, dtype=np.float32)
    w = {k: bf(v) for k, v in w.items()}
    names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "g": "g_proj", "q.norm": "q_norm", "k.norm": "k_norm"}
    want = set(type(mixer).param_shapes(spec))
    mixer.load({names[k]: dev(v, dtype) for k, v in w.items() if names[k] in want}, dtype, DEV)
    return mixer, f64(w)


def test_the_slopes_fall_by_a_constant_factor_down_to_one_in_256():
    from quicknn_b200.config.mubasun import distance_slopes
    for H in (1, 2, 3, 4, 5, 8, 12):
        got = np.array(distance_slopes(H))
        assert np.allclose(got, MP.slopes(H), rtol=1e-12) and np.isclose(got[-1], 1 / 256)
        assert np.allclose(got[1:] / got[:-1], 2.0 ** (-8.0 / H))


@pytest.mark.parametrize("dtype,H,G,d,dv,window", [
    (torch.float32, 4, 2, 16, 24, None), (torch.float32, 2, 1, 24, 8, 9), (torch.float32, 4, 4, 12, 20, 64),
    (torch.float32, 6, 2, 20, 12, 65), (torch.float32, 1, 1, 64, 64, 1), (torch.float32, 4, 2, 32, 32, 63),
    (torch.float32, 3, 1, 8, 8, 140), (torch.float32, 8, 1, 16, 16, 20), (torch.float32, 12, 2, 8, 12, None),
    (torch.bfloat16, 4, 1, 64, 40, None), (torch.bfloat16, 4, 2, 64, 64, 70), (torch.bfloat16, 2, 1, 96, 80, 44),
    (torch.bfloat16, 8, 4, 128, 64, 130), (torch.bfloat16, 4, 2, 24, 40, 7), (torch.bfloat16, 8, 2, 64, 64, 137),
    (torch.bfloat16, 16, 2, 64, 64, 100), (torch.bfloat16, 6, 1, 128, 128, None)])
def test_attention_alone_and_a_window_or_a_slope_one_off_would_show(dtype, H, G, d, dv, window):
    """A prompt longer than the window and two pages, then 70 tokens one by one across a page edge and the ring, then
    a portion.  In float32 the scores are scaled until attention is nearly one-hot, so that a window one token off, a
    key at the wrong page, the slopes of the wrong heads or a bias by the key's place alone would move the output."""
    from quicknn_b200.cache import KVCache
    W = 64
    sharp = dtype == torch.float32
    m = _att(H, G, d, dv, 1.5 if sharp else 0.3, window=window)
    mixer, w = _attention_mixer(W, m, dtype, 100)
    need = mixer.cache_need()
    D = d if d == dv and d % 8 == 0 else (max(d, dv) + 7) // 8 * 8
    assert (need.n_kv_heads, need.head_dim, need.window) == (G, D, window)
    n, single, portion = 150, 70, 6
    x = bf(rnd((n + single + portion, W), 7))
    ref, _ = MP.attention(x.astype(np.float64), w, m, 1e-5)
    if sharp:
        if window is not None and window > 1:
            off, _ = MP.attention(x.astype(np.float64), w, dict(m, mask={"size": window - 1}), 1e-5)
            assert np.abs(off - ref).max() > 0.02 * np.abs(ref).max()      # a thousand times the tolerance below
        if H > 1 and (window is None or window > 8):        # the heads' slopes in the other order
            import unittest.mock
            with unittest.mock.patch.object(MP, "slopes", lambda heads: 2.0 ** (-8.0 * (heads - np.arange(heads)) / heads)):
                off, _ = MP.attention(x.astype(np.float64), w, m, 1e-5)
            assert np.abs(off - ref).max() > 0.05 * np.abs(ref).max()
    cache = KVCache([need], [None], 1024, 2, 512, dtype, DEV)
    s = cache.allocate()
    tol = (3e-5 if sharp else 0.03) * max(1.0, np.abs(ref).max())
    step = part_step([n], [0], [s], "prefill", dtype, cache, mixer)
    assert np.abs(host(mixer.forward(dev(x[:n], dtype), step, cache.line(0))) - ref[:n]).max() < tol
    for t in range(n, n + single):
        step = part_step([1], [t], [s], "decode", dtype, cache, mixer)
        y = host(mixer.forward(dev(x[t:t + 1], dtype), step, cache.line(0)))
        assert np.abs(y - ref[t:t + 1]).max() < tol, f"position {t}"
    t = n + single
    step = part_step([portion], [t], [s], "extend", dtype, cache, mixer)
    step.whole = None
    assert np.abs(host(mixer.forward(dev(x[t:], dtype), step, cache.line(0))) - ref[t:]).max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_that_one_score_singles_out(dtype):
    """Among 600 keys the third one is made to match the last query as well as the last row's own key does (every head's
    query matrix is its key matrix, and the norms make a row's size irrelevant to its direction), while its value is
    five times the last row's own.  The distance costs it 2.3 in the last head and 37 in the first: without a window
    the far value shows in the last head's output and is absent from the first head's; with a window of 500 it is
    absent from both; the kernels give the plain result in every case."""
    from quicknn_b200.cache import KVCache
    W, H, G, d, dv, n = 32, 2, 1, 32, 16, 600
    outs = {}
    for window in (None, 500):
        m = _att(H, G, d, dv, 0.6, window=window)          # |q| = |k| = sqrt(32): a matching pair scores 0.6 * 32 = 19.2
        mixer, w = _attention_mixer(W, m, dtype, 200, tie_qk=True)
        w["g"][:] = 0.0                                       # the gate at one half everywhere
        mixer.w_out_gate.zero_()
        x = bf(rnd((n, W), 8, 0.3))
        x[2] = bf(5.0 * rnd(W, 9))
        x[-1] = bf(x[2] / 5.0)
        ref, _ = MP.attention(x.astype(np.float64), w, m, 1e-5)
        heads = (ref[-1] @ np.linalg.pinv(w["o"]).T).reshape(H, dv)
        outs[window] = heads
        cache = KVCache([mixer.cache_need()], [None], 1024, 1, 1024, dtype, DEV)
        s = cache.allocate()
        step = part_step([n - 1], [0], [s], "prefill", dtype, cache, mixer)
        mixer.forward(dev(x[:n - 1], dtype), step, cache.line(0))
        step = part_step([1], [n - 1], [s], "decode", dtype, cache, mixer)
        y = host(mixer.forward(dev(x[n - 1:], dtype), step, cache.line(0)))
        assert np.abs(y - ref[-1:]).max() < (3e-5 if dtype == torch.float32 else 0.03) * max(1.0, np.abs(ref).max())
    far, near_ = outs[None], outs[500]
    assert np.abs(far[1] - near_[1]).max() > 0.15 * np.abs(far[1]).max()      # slope 1/256: 597 steps cost 2.3
    assert np.abs(far[0] - near_[0]).max() < 1e-6 * np.abs(far[0]).max()      # slope 1/16: 597 steps cost 37


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_inside_a_long_prompt(dtype):
    """The same far key, met by the last row of a whole prompt and by the last row of a portion of 40."""
    from quicknn_b200.cache import KVCache
    W, H, G, d, dv, n = 32, 2, 1, 32, 16, 600
    m = _att(H, G, d, dv, 0.6)
    mixer, w = _attention_mixer(W, m, dtype, 210, tie_qk=True)
    x = bf(rnd((n, W), 8, 0.3))
    x[2] = bf(5.0 * rnd(W, 9))
    x[-1] = bf(x[2] / 5.0)
    ref, _ = MP.attention(x.astype(np.float64), w, m, 1e-5)
    lost, _ = MP.attention(x[3:].astype(np.float64), w, m, 1e-5)
    assert np.abs(lost[-1] - ref[-1]).max() > 0.05 * np.abs(ref[-1]).max()
    tol = (3e-5 if dtype == torch.float32 else 0.03) * max(1.0, np.abs(ref).max())
    cache = KVCache([mixer.cache_need()], [None], 2048, 2, 1024, dtype, DEV)
    a, b = cache.allocate(), cache.allocate()
    step = part_step([n], [0], [a], "prefill", dtype, cache, mixer)
    assert np.abs(host(mixer.forward(dev(x, dtype), step, cache.line(0))) - ref).max() < tol
    step = part_step([n - 40], [0], [b], "prefill", dtype, cache, mixer)
    mixer.forward(dev(x[:n - 40], dtype), step, cache.line(0))
    step = part_step([40], [n - 40], [b], "extend", dtype, cache, mixer)
    step.whole = None
    assert np.abs(host(mixer.forward(dev(x[n - 40:], dtype), step, cache.line(0))) - ref[n - 40:]).max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_first_tokens_and_a_slot_that_is_handed_out_again(dtype):
    """Sequences of one, two and three tokens (the first row attends to itself alone, whatever is in the pages), then a
    sequence in the slot and pages that a longer one has just given back."""
    from quicknn_b200.cache import KVCache
    W = 48
    m = _att(4, 2, 16, 16, 0.5, window=5)
    mixer, w = _attention_mixer(W, m, dtype, 220)
    tol = 3e-5 if dtype == torch.float32 else 0.03
    cache = KVCache([mixer.cache_need()], [None], 512, 2, 256, dtype, DEV)
    long = bf(rnd((140, W), 1, 3.0))
    s = cache.allocate()
    mixer.forward(dev(long, dtype), part_step([140], [0], [s], "prefill", dtype, cache, mixer), cache.line(0))
    cache.free(s)
    for n in (1, 2, 3):
        x = bf(rnd((n + 8, W), 10 + n))
        ref, _ = MP.attention(x.astype(np.float64), w, m, 1e-5)
        s = cache.allocate()
        got = host(mixer.forward(dev(x[:n], dtype), part_step([n], [0], [s], "prefill", dtype, cache, mixer), cache.line(0)))
        assert np.abs(got - ref[:n]).max() < tol * max(1.0, np.abs(ref).max())
        for t in range(n, n + 8):
            step = part_step([1], [t], [s], "decode", dtype, cache, mixer)
            y = host(mixer.forward(dev(x[t:t + 1], dtype), step, cache.line(0)))
            assert np.abs(y - ref[t:t + 1]).max() < tol * max(1.0, np.abs(ref).max()), f"{n} tokens, then position {t}"
        cache.free(s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("own,other", [(None, 21), (9, 40), (70, 70), (33, None)])
def test_a_layer_on_another_layers_keys_with_a_window_of_its_own(dtype, own, other):
    """Two mixers over one cache line: the second has queries, a gate and a window of its own, and neither keys nor
    values.  Prompts of unequal lengths, single tokens, a portion."""
    import dataclasses
    from quicknn_b200.cache import KVCache
    W = 48
    d = 64 if dtype == torch.bfloat16 else 16
    m1, m2 = _att(4, 2, d, 24, 0.4, window=own), _att(4, 2, d, 24, 0.3, window=other)
    owner, w1 = _attention_mixer(W, m1, dtype, 300)
    reader, w2 = _attention_mixer(W, m2, dtype, 400, shared=True)
    shapes = type(reader).param_shapes(reader.spec)
    assert not {"k_proj", "v_proj", "k_norm"} & set(shapes) and {"q_proj", "q_norm", "g_proj", "o_proj"} <= set(shapes)
    lens, more = [70, 5, 129], 70      # the continued step overruns a ring of 64
    xs = [bf(rnd((n + more, W), 30 + i)) for i, n in enumerate(lens)]
    ys = [bf(rnd((n + more, W), 40 + i)) for i, n in enumerate(lens)]          # the reader's input differs from the owner's
    refs = []
    for x, y in zip(xs, ys):
        _, kv = MP.attention(x.astype(np.float64), w1, m1, 1e-5)
        refs.append(MP.attention(y.astype(np.float64), w2, m2, 1e-5, kv=kv)[0])
    need = owner.cache_need()
    if need.window is not None and (other is None or other > need.window):   # the line keeps what its widest reader sees
        need = dataclasses.replace(need, window=other)
    cache = KVCache([need], [None], 1024, 3, 512, dtype, DEV)
    slots = [cache.allocate() for _ in lens]
    tol = (3e-5 if dtype == torch.float32 else 0.03) * max(1.0, max(np.abs(r).max() for r in refs))

    def both(mode, counts, starts, who):
        step = part_step(counts, starts, [slots[i] for i in who], mode, dtype, cache, owner)
        step.whole = None
        line = cache.line(0, writes=True)
        line.has_readers = True
        owner.forward(dev(np.concatenate([xs[i][s:s + c] for i, s, c in zip(who, starts, counts)]), dtype), step, line)
        got = host(reader.forward(dev(np.concatenate([ys[i][s:s + c] for i, s, c in zip(who, starts, counts)]), dtype), step,
                                  cache.line(0, writes=False)))
        for call in step.after_layers:                 # the owner's append of a continued step waits for its readers
            call()
        step.after_layers.clear()
        want = np.concatenate([refs[i][s:s + c] for i, s, c in zip(who, starts, counts)])
        assert np.abs(got - want).max() < tol, mode
    both("prefill", lens, [0, 0, 0], [0, 1, 2])
    both("decode", [1, 1, 1], lens, [0, 1, 2])
    both("extend", [more - 3, 2], [lens[0] + 1, lens[2] + 1], [0, 2])
    both("decode", [1, 1], [lens[0] + more - 2, lens[2] + 3], [0, 2])


# ---- whole models -----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("A", "bfloat16", False), ("B", "float32", True),
                                              ("B", "bfloat16", False), ("C", "float32", True), ("C", "bfloat16", False),
                                              ("B", "float32", False)])
def test_every_cutting_gives_the_plain_logits(muba, tmp_path, whole_model_tolerance, name, dtype, peaky):
    folder, plain = muba(name, dtype, peaky)
    requests = prompts(name, LENGTHS_B if name == "B" else LENGTHS)
    ref = [plain.logits(t) for t in requests]
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if name == "B" else 384)
    try:
        worst = run_all_cuttings(replay, requests, ref, dtype)
    finally:
        replay.close()
    print(f"mubasun {name} {dtype} peaky={peaky}: largest error {worst:.3g}")


def test_the_stream_after_every_layer(muba):
    """float32, layer by layer: what each block leaves in the stream is the plain implementation's."""
    from quicknn_b200.engine import Engine, Model
    for name in ("A", "B", "C"):
        folder, plain = muba(name, "float32", True)
        toks = prompts(name, [90], seed=11)[0]
        want = plain.residual_stream(toks)[1:]
        model = Model.from_folder(folder, "float32", DEV)
        seen = []
        for blk in model.blocks:
            def wrapped(resid, step, line, normed=None, next_norm=None, _inner=blk.forward):
                out = _inner(resid, step, line, normed=normed, next_norm=next_norm)
                seen.append(host(out[0] if isinstance(out, tuple) else out))
                return out
            blk.forward = wrapped
        eng = Engine(model, max_tokens=256)
        eng.step([(eng.new_sequence(), toks)], "last")
        assert len(seen) == len(want)
        for i, (g, r) in enumerate(zip(seen, want)):
            assert np.abs(g - r).max() < 3e-5 * max(1.0, np.abs(r).max()), f"model {name}, layer {i}"


@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("B", "float32", True), ("B", "bfloat16", False),
                                              ("A", "bfloat16", False), ("C", "float32", True)])
def test_prompts_in_portions_down_to_two_tokens(muba, tmp_path, name, dtype, peaky):
    """Steps that continue sequences by several tokens, beside requests that join or sit out."""
    folder, plain = muba(name, dtype, peaky)
    big = name == "B"
    requests = prompts(name, [257, 170, 45] if big else [129, 70, 45], seed=7)
    ref = [plain.logits(t) for t in requests]
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if big else 384)
    pos = [0, 0, 0]

    def step(*parts, end=()):
        entries = [(f"r{i}", requests[i][pos[i]:pos[i] + n], range(n)) for i, n in parts]
        got = replay.step(entries, end=[f"r{i}" for i in end])
        r = 0
        for i, n in parts:
            ok, err, tol = near(got[r:r + n], ref[i][pos[i]:pos[i] + n], dtype)
            assert ok, f"request {i} positions {pos[i]}..{pos[i] + n - 1}: error {err:.3g} > {tol:.3g}"
            pos[i] += n
            r += n
    try:
        a, b = len(requests[0]), len(requests[1])
        step((0, 2), (1, 62))
        step((0, 62))                            # request 1 sits out; request 0 reaches the page edge
        step((0, 2), (1, 2), (2, 40))            # portions of two across the edge; request 2 joins
        step((0, 1), (1, 1), (2, 1))
        step((0, a - 67 - 3), (2, 4), end=[2])   # a portion longer than the windows
        step((0, 3), (1, b - 65), end=[0, 1])
        assert pos == [a, b, 45]
        got = replay.step([("again", requests[0], [a - 1])], end=["again"])      # what they held is free again
        ok, err, tol = near(got, ref[0][a - 1:a], dtype)
        assert ok, (err, tol)
    finally:
        replay.close()


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(muba, name):
    """More requests than slots, so that slots and pages are handed out again; decode steps run from CUDA graphs, one
    step ahead of the host; the tokens are the plain implementation's."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = muba(name, "float32", True)
    reqs = prompts(name, [5, 70, 1, 33, 12], seed=3)
    llm = LLM(folder, max_context=256, max_batch=2, dtype="float32")
    res = llm.generate(reqs, GenerationOptions.greedy(12), stop_ids=[])
    for r, p in zip(res, reqs):
        seq = list(p)
        for t in r.tokens:                      # the best token at its place (a tie within rounding may go either way)
            row = plain.logits(seq)[-1]
            assert row[t] >= row.max() - 1e-4 * max(1.0, np.abs(row).max()), f"request {r.index}"
            seq.append(t)
    llm16 = LLM(folder, max_context=256, max_batch=4, dtype="bfloat16")
    for r, p in zip(llm16.generate(reqs, GenerationOptions.greedy(6), stop_ids=[]), reqs):
        seq = list(p)
        for t in r.tokens:                      # bfloat16: every token is at least a near-best one of the plain logits
            row = plain.logits(seq)[-1]
            assert row[t] >= row.max() - 0.1 * max(1.0, np.abs(row).max())
            seq.append(t)


def test_long_decoding_passes_windows_and_page_edges(muba):
    """150 tokens generated one by one after a short prompt: the windows of 9 and 33 and the ring of a page pass over
    decoded tokens, the readers see what their owners appended."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = muba("A", "float32", True)
    p = prompts("A", [3], seed=9)[0]
    llm = LLM(folder, max_context=256, max_batch=1, dtype="float32")
    got = llm.generate([p], GenerationOptions.greedy(150), stop_ids=[])[0].tokens
    seq = p + got
    ref = plain.logits(seq[:-1])
    for i, t in enumerate(got):
        row = ref[len(p) - 1 + i]
        assert row[t] >= row.max() - 1e-4 * max(1.0, np.abs(row).max()), f"token {i}"


def test_the_command_line_serves_the_design(muba, tmp_path):
    import subprocess
    import sys
    from conftest import ROOT

    def run(*argv):
        return subprocess.run([sys.executable, "-m", "quicknn_b200", *argv], cwd=ROOT, capture_output=True, text=True)
    folder, plain = muba("A", "float32", True)
    r = run("info", "--model", folder)
    assert r.returncode == 0, r.stderr
    info = json.loads(r.stdout)
    assert info["architecture"] == "Mubasun" and info["layers"] == len(MUBA_A["layers"])
    p = prompts("A", [9, 4], seed=5)
    r = run("generate", "--model", folder, "--prompt-ids", ";".join(",".join(map(str, q)) for q in p), "--max-new-tokens", "8",
            "--temperature", "0", "--dtype", "float32", "--max-context", "64", "--stop-ids", "")
    assert r.returncode == 0, r.stderr
    got = [json.loads(l) for l in r.stdout.splitlines() if l.strip()]
    assert [g["tokens"] for g in got] == [plain.greedy(q, 8) for q in p]
    # a model folder with random weights from a configuration file, and its replay
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(MUBA_C))
    out = tmp_path / "random_c"
    r = run("random", "--config", str(cfg), "--seed", "3", "--out", str(out), "--dtype", "bfloat16")
    assert r.returncode == 0, r.stderr
    ref = MP.PlainMubasun(str(out))
    toks = prompts("C", [21], seed=6)[0]
    replay = Replay(str(out), "float32", tmp_path / "logits", max_tokens=64)       # bfloat16 weights, widened exactly
    try:
        got = replay.step([("x", toks, range(len(toks)))], end=["x"])
    finally:
        replay.close()
    ok, err, tol = close(got, ref.logits(toks), "float32")
    assert ok, (err, tol)


def _prompts_then_single_tokens(folder, plain, reqs, lens, extra, dtype, max_tokens, what, float32=1e-4):
    from quicknn_b200.engine import Engine, Model
    ref = [plain.logits(t) for t in reqs]
    eng = Engine(Model.from_folder(folder, dtype, DEV), max_tokens=max_tokens)
    slots = [eng.new_sequence() for _ in reqs]
    got = eng.step([(s, t[:n]) for s, t, n in zip(slots, reqs, lens)], "all").cpu().numpy()
    at = 0
    for r, n in zip(ref, lens):
        ok, err, tol = near(got[at:at + n], r[:n], dtype, float32)
        assert ok, f"{what} {dtype}: prompt of {n}: error {err:.3g} > {tol:.3g}"
        at += n
    for t in range(extra):
        got = eng.step([(s, [q[n + t]]) for s, q, n in zip(slots, reqs, lens)], "last").cpu().numpy()
        for i, (r, n) in enumerate(zip(ref, lens)):
            ok, err, tol = near(got[i:i + 1], r[n + t:n + t + 1], dtype, float32)
            assert ok, f"{what} {dtype}: request {i} decoded token {t}: error {err:.3g} > {tol:.3g}"
    for s in slots:
        eng.release(s)
    eng.cache.audit()


def test_layer_sizes_that_take_the_tensor_core_kernels(tmp_path):
    """Head size 128 (the tcgen05 prompt attention and the tensor-core decode attention with the distance bias, also for
    the layers on shared keys and values and for values carried wider than they are), products of several hundred rows
    (the tcgen05 GEMMs with xIELU and the gate in their epilogues, the grouped expert products), prompts long enough for
    a window to pass inside a prompt; then single tokens."""
    att = _att(8, 2, 128, 64, 0.09, window=300)
    raw = dict(architecture="Mubasun", vocab=1000, width=512, max_positions=1024, norm={"eps": 1e-5, "groups": 8},
               initializer_range=0.04,
               layers=[_layer(_att(4, 2, 128, 128, 0.1), _dense(1024)),
                       _layer(att, _moe(256, 8, 1, 2, 1.5, shared=384)),
                       _layer(dict(att, kv_from=1, mask={"size": 130}), _moe(128, 4, 0, 1, 1.0)),
                       _layer(dict(_att(4, 2, 128, 128, 0.08), kv_from=0), _dense(768))])
    CONFIGS["L"] = (raw, 21)
    lens, extra = [600, 130], 3
    reqs = prompts("L", [n + extra for n in lens], seed=4)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path, "L", dtype, False)
        _prompts_then_single_tokens(folder, MP.PlainMubasun(folder), reqs, lens, extra, dtype, 2048, "layer sizes")


def test_long_prompts_with_windows_that_pass_inside_them_and_over_decoded_tokens(tmp_path):
    """Prompts of 1200 and 300 tokens, then 40 single tokens: windows of 150 and 300 and a reader without one."""
    att = _att(6, 2, 32, 32, 0.2, window=150)
    raw = dict(architecture="Mubasun", vocab=700, width=96, max_positions=1300, norm={"eps": 1e-5, "groups": 3},
               initializer_range=0.08,
               layers=[_layer(att, _dense(160)),
                       _layer(dict(att, kv_from=0, mask={"size": 300}), _moe(48, 6, 1, 2, 1.4, shared=64)),
                       _layer(_att(4, 1, 64, 64, 0.15), _moe(32, 4, 2, 3, 0.9)),
                       _layer({k: v for k, v in dict(att, kv_from=0).items() if k != "mask"}, _dense(96))])
    CONFIGS["F"] = (raw, 41)
    lens, extra = [1200, 300], 40
    reqs = prompts("F", [n + extra for n in lens], seed=12)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path, "F", dtype, False)
        _prompts_then_single_tokens(folder, MP.PlainMubasun(folder), reqs, lens, extra, dtype, 4096, "long prompts")


def test_odd_sizes_everywhere(tmp_path):
    """A width, head sizes, inner widths and a vocabulary that are odd numbers."""
    raw = dict(architecture="Mubasun", vocab=131, width=39, max_positions=128, norm={"eps": 1e-5, "groups": 3},
               initializer_range=0.1,
               layers=[_layer(_att(3, 1, 5, 7, 0.4, window=11), _dense(45)),
                       _layer(_att(2, 2, 9, 3, 0.3), _moe(11, 3, 1, 2, 1.1, shared=13)),
                       _layer(_att(6, 1, 5, 7, 0.25, kv_from=0), _moe(7, 2, 0, 1, 0.9))])
    CONFIGS["O"] = (raw, 31)
    lens, extra = [70, 3], 4
    reqs = prompts("O", [n + extra for n in lens], seed=8)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path, "O", dtype, False)
        _prompts_then_single_tokens(folder, MP.PlainMubasun(folder), reqs, lens, extra, dtype, 512, "odd sizes")


# ---- configurations drawn at random ---------------------------------------------------------------------------------

def random_config(seed):
    """Every size, the order of the layers and every constant drawn from a seed."""
    rng = np.random.default_rng(3000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]  # noqa: E731
    groups = pick([1, 2, 4, 5])
    width = groups * pick([8, 12, 16, 20, 32])

    def mixer():
        G = pick([1, 2, 3])
        return _att(G * pick([1, 2, 4]), G, pick([8, 12, 16, 24, 32, 64]), pick([8, 16, 20, 32, 64]),
                    float(rng.uniform(0.1, 0.4)), window=pick([None, 1, 3, 17, 63, 64, 65, 80, 140]))

    def mlp():
        kind = pick([None, "dense", "moe", "moe"])
        if kind is None:
            return None
        if kind == "dense":
            return _dense(pick([32, 72, 128]))
        experts, identity = int(rng.integers(1, 9)), int(rng.integers(0, 4))
        return _moe(pick([8, 24, 64]), experts, identity, int(rng.integers(1, min(4, experts + identity) + 1)),
                    float(rng.uniform(0.5, 3.0)), shared=pick([None, 16, 40]))
    layers, owners = [], []
    for i in range(int(rng.integers(1, 7))):
        if owners and rng.random() < 0.4:
            j = pick(owners)
            m = dict(layers[j]["mixer"], kv_from=j, heads=layers[j]["mixer"]["kv_heads"] * pick([1, 2, 4]),
                     scale=float(rng.uniform(0.1, 0.4)))
            m.pop("mask", None)
            size = pick([None, 2, 9, 64, 70, 150])
            if size is not None:
                m["mask"] = {"size": size}
            layers.append(_layer(m, mlp()))
        else:
            owners.append(i)
            layers.append(_layer(mixer(), mlp()))
    return dict(architecture="Mubasun", vocab=int(rng.integers(100, 700)), width=width, max_positions=256,
                norm={"eps": pick([1e-5, 1e-6]), "groups": groups}, initializer_range=0.07, layers=layers)


@pytest.mark.parametrize("seed", range(24))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Prompts of unequal lengths in one step, then tokens one by one, against the plain logits: float32 sharply for
    every configuration, bfloat16 for every other one."""
    raw = random_config(seed)
    name = f"R{seed}"
    CONFIGS[name] = (raw, 50 + seed)
    lens, extra = [130, 7, 1, 70], 5
    reqs = prompts(name, [n + extra for n in lens], seed=seed)
    for dtype in (("float32", "bfloat16") if seed % 2 == 0 else ("float32",)):
        folder = make_folder(tmp_path, name, dtype, dtype == "float32")
        _prompts_then_single_tokens(folder, MP.PlainMubasun(folder), reqs, lens, extra, dtype, 1024,
                                    f"seed {seed} ({raw['layers']})", 3e-4)
