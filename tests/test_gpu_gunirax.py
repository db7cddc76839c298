"""Gunirax on the GPU against the plain implementation (tests/plain/gunirax_plain.py): the small kernels (dynamic tanh
alone, after an add, with the embedding; the bounded forget gates; bias, rotation, norm and keys copied as values); the
router with groups and experts without a gate; the sigmoid attention mixer alone over a cache of its own (prompts,
single tokens across page, ring and chunk edges, a portion, a slot handed out again, a key that stands out just inside
and just outside a chunk and far back); the two matrix memories alone; then whole models through bin/trace_run under
every cutting, in portions down to two tokens, through the entry point's generation loop, the command line, and
configurations drawn at random.  The configurations are small and differ from one another in every size and constant."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import close
from plain import gunirax_plain as GP
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


ROUTED_RUNS = [0]         # executed layers with routed experts in the model that is being compared (set by `routed_runs`)


def routed_runs(raw):
    """How often a step of this configuration routes: the executed layers (a looped layer counts every pass) whose
    feed-forward has a router.  Remembered for `near`."""
    n = sum(1 for r in GP.layer_runs(raw) if (raw["layers"][r["layer"]].get("mlp") or {}).get("kind") == "moe")
    ROUTED_RUNS[0] = n
    return n


def near(got, ref, dtype, float32=1e-4):
    """How whole models are compared.  float32: the largest difference, 1e-4 of the largest logit; that is the sharp
    check: a wrong mask, key, chunk edge, state or expert moves these models' logits by 1e-2 and more.  bfloat16: a row is
    compared by the root mean square of its difference (mean taken off) against that of the logits, at most a tenth,
    and some rows may lie beyond, one in thirty for the model and as many again for every executed layer that routes:
    a router sees the bfloat16 rounding of its input and chooses another expert, or another group, where two ranking
    values lie within rounding of each other, and that row then differs by an expert's whole output; a looped stack
    routes in every pass."""
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
    allowed = max(1, len(e) * (1 + ROUTED_RUNS[0]) // 30)
    return over <= allowed, float(np.sort(e)[-1 - min(over, allowed, len(e) - 1)]), 0.1


@pytest.fixture
def whole_model_tolerance(monkeypatch):
    import test_gpu_replay
    monkeypatch.setattr(test_gpu_replay, "close", near)


# ---- configurations -------------------------------------------------------------------------------------

def _left(heads, kv, dim, scale, chunk, dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _par(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _hgrn(heads, dim, vdim, mlp):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, scale, count, keep, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


# A: a recurrent layer first; the loop covers the two middle layers three times; a chunk shorter than a page and one of
#    a single position; partly rotated heads; a layer without a feed-forward; groups of one expert
GUNI_A = dict(architecture="Gunirax", vocab=300, width=64, embedding={"scale": 2.5}, norm={"eps": 1e-6},
              loop={"start": 1, "stop": 3, "times": 3}, initializer_range=0.08, layers=[
                  _hgrn(2, 16, 24, _dense(96)),
                  _par(_left(4, 2, 16, 0.3, 9, 8, 1000.0, (8.0, 1.0, 4.0, 64)), _right(2, 8, 24, (0.6, 0.98)),
                       _moe(24, 6, 2, 1.7, 6, 3, shared=40)),
                  _par(_left(2, 2, 24, 0.2, 1, 24), _right(3, 16, 8, (0.9, 0.5, 1.0)), None),
                  _hgrn(1, 40, 12, _moe(16, 4, 3, 0.8, 2, 2))])
# B: head size 64, a chunk beyond a page, no loop at all, one kv head, every group kept, top 1, no shared expert in one
#    routed layer, a left branch without a mask
GUNI_B = dict(architecture="Gunirax", vocab=512, width=128, embedding={"scale": 1.0}, norm={"eps": 1e-5},
              initializer_range=0.06, layers=[
                  _par(_left(4, 1, 64, 0.11, 70, 64, 30000.0, (4.0, 1.0, 4.0, 128)), _right(2, 32, 64, (0.8, 0.999)),
                       _moe(64, 8, 1, 1.0, 4, 4, shared=96)),
                  _hgrn(2, 64, 32, _dense(192)),
                  _par(_left(2, 2, 64, 0.13, 130, 32), _right(1, 64, 128, (0.95,)), _moe(32, 4, 2, 2.0, 2, 1)),
                  _par(_left(4, 2, 32, 0.2, None, 16), _right(4, 16, 16, (0.7, 0.8, 0.9, 0.99)), _dense(64))])
# C: a width, head sizes and a vocabulary that are no multiple of 8, the loop over everything, twice; one head
#    everywhere in one layer; every expert chosen; a chunk of exactly a page
GUNI_C = dict(architecture="Gunirax", vocab=301, width=100, embedding={"scale": 0.7}, norm={"eps": 1e-4},
              loop={"start": 0, "stop": 3, "times": 2}, initializer_range=0.07, layers=[
                  _par(_left(5, 5, 12, 0.3, 64, 6, 500.0), _right(5, 4, 20, (0.5, 0.6, 0.7, 0.8, 0.9)), _dense(70)),
                  _par(_left(1, 1, 20, 0.22, 33, 20, 20000.0, (2.0, 1.0, 2.0, 32)), _right(1, 12, 28, (0.97,)),
                       _moe(36, 3, 3, 3.0, 1, 1, shared=20)),
                  _hgrn(3, 4, 28, _moe(12, 9, 4, 0.5, 3, 2))])
CONFIGS = {"A": (GUNI_A, 3), "B": (GUNI_B, 4), "C": (GUNI_C, 5)}
LENGTHS = [70, 33, 129, 45, 100, 64]
LENGTHS_B = [170, 33, 257, 45, 100, 64]


def make_folder(base, name, storage, peaky):
    """Random weights, with what random draws would leave trivial set by hand: the mixing matrices near the identity
    with sizeable other entries, lower bounds of the forget gates spread over [0, 0.95], corrections a fifth of the
    spread of the scores; ``peaky`` scales the router's matrix so that choices are clear."""
    from quicknn_b200.config import GUNIRAX, GuniraxConfig
    from quicknn_b200.weights import random_tensors, write_safetensors
    raw, seed = CONFIGS[name]
    cfg = GuniraxConfig.from_dict(raw)
    d = os.path.join(str(base), f"guni{name}_{storage}{'_peaky' if peaky else ''}")
    os.makedirs(d, exist_ok=True)
    tensors = dict(random_tensors(GUNIRAX, cfg, seed, torch.float32, 0.2))
    for k in list(tensors):
        t = tensors[k]
        if k.endswith(".talk"):
            tensors[k] = torch.eye(t.shape[0]) + t * 4.0
        elif k.endswith(".lower"):
            tensors[k] = torch.linspace(0.0, 0.95, t.numel())
        elif k.endswith("mlp.correction"):
            tensors[k] = t * 0.2
        elif k.endswith(".alpha"):
            tensors[k] = t * 0.6
        elif peaky and k.endswith("mlp.router"):
            tensors[k] = t * 4.0
    dt = torch.float32 if storage == "float32" else torch.bfloat16
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(d, "model.safetensors"), {k: v.to(dt) for k, v in tensors.items()})
    return d


@pytest.fixture(scope="module")
def guni(tmp_path_factory):
    base = tmp_path_factory.mktemp("gunirax")
    made = {}

    def get(name, storage="float32", peaky=False):
        key = (name, storage, peaky)
        if key not in made:
            folder = make_folder(base, name, storage, peaky)
            made[key] = (folder, GP.PlainGunirax(folder))
        return made[key]
    return get


def prompts(name, lengths, seed=0):
    rng = np.random.default_rng(100 + seed)
    return [rng.integers(1, CONFIGS[name][0]["vocab"], n).tolist() for n in lengths]


# ---- the small kernels ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_alone_after_an_add_and_with_the_embedding(dtype):
    from quicknn_b200.kernels import ops
    tol = 2e-6 if dtype == torch.float32 else 0.01
    for rows, width in ((3, 100), (70, 64), (5, 2304), (2, 37)):
        x, w, b = bf(rnd((rows, width), 1, 2.0) + 0.3), bf(rnd(width, 2, 0.2) + 1.0), bf(rnd(width, 3, 0.3))
        named = {"n": w.astype(np.float64), "n.b": b.astype(np.float64), "n.alpha": np.float64(0.625)}
        ref = GP.dynamic_tanh(x.astype(np.float64), named, "n")
        for src in (dev(x, dtype), dev(x)):                  # rows of either type
            assert np.abs(host(ops.dyt(src, 0.625, dev(w, dtype), dev(b, dtype), dtype)) - ref).max() < tol * np.abs(ref).max()
        resid, a, c = rnd((rows, width), 4, 3.0), bf(rnd((rows, width), 5)), rnd((rows, width), 6, 2.0)
        for first, second in ((a, None), (None, c), (a, c)):
            r = dev(resid)
            normed = ops.add_dyt(r, None if first is None else dev(first, dtype), None if second is None else dev(second),
                                 0.625, dev(w, dtype), dev(b, dtype), dtype)
            want = resid.astype(np.float64) + (0 if first is None else first) + (0 if second is None else second)
            assert np.abs(host(r) - want).max() < 3e-6 * np.abs(want).max()          # the stream itself is float32
            assert np.abs(host(normed) - GP.dynamic_tanh(want, named, "n")).max() < tol * np.abs(ref).max()
        r = dev(resid)
        assert ops.add_dyt(r, dev(a, dtype)) is None                                 # the last layer: no norm follows
        assert np.abs(host(r) - (resid.astype(np.float64) + a)).max() < 3e-6 * np.abs(resid).max()
    V, width = 50, 72
    table, w, b = bf(rnd((V, width), 7)), bf(rnd(width, 8, 0.2) + 1.0), bf(rnd(width, 9, 0.3))
    tokens = np.array([0, 49, 7, 7, 3], dtype=np.int32)
    x, normed = ops.embed_dyt(torch.tensor(tokens, device=DEV), dev(table, dtype), 1.5, 0.8, dev(w, dtype), dev(b, dtype), dtype)
    want = table[tokens].astype(np.float64) * 1.5
    assert x.dtype == torch.float32 and np.abs(host(x) - want).max() < 1e-6 * np.abs(want).max()
    ref = np.tanh(0.8 * want) * w + b
    assert np.abs(host(normed) - ref).max() < tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_of_the_queries_and_forget_gates_with_a_lower_bound(dtype):
    from quicknn_b200.kernels import ops
    T, nq, nf, spare = 9, 24, 24, 5
    rows = bf(rnd((T, spare + nq + nf + 7), 1, 2.0))
    bias, lower = bf(rnd(nf, 2)), bf(np.linspace(0.0, 1.0, nf))
    t = dev(rows, dtype)
    f = ops.bounded_gates(t, spare, nq, spare + nq, nf, dev(bias, dtype), dev(lower, dtype))
    z = rows[:, spare + nq:spare + nq + nf].astype(np.float64)
    want = lower + (1 - lower.astype(np.float64)) * GP.sigmoid(z + bias)
    assert f.dtype == torch.float32 and np.abs(host(f) - want).max() < 1e-6
    got = host(t)
    q = rows[:, spare:spare + nq].astype(np.float64)
    assert np.abs(got[:, spare:spare + nq] - GP.silu(q)).max() < (1e-6 if dtype == torch.float32 else 0.02)
    keep = np.ones(rows.shape[1], dtype=bool)
    keep[spare:spare + nq] = False
    assert (got[:, keep] == rows[:, keep]).all()             # nothing else is touched


@pytest.mark.parametrize("hd,rot,nq,nk", [(16, 8, 3, 1), (24, 24, 4, 2), (12, 6, 5, 5), (64, 64, 4, 1), (128, 32, 2, 2), (8, 0, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_rotation_then_a_norm_without_weights_and_keys_copied_as_values(hd, rot, nq, nk, dtype):
    """The rows hold queries and keys; the destination gets q | k | v with v the keys after the bias alone."""
    from quicknn_b200.kernels import ops
    T, eps, spare = 7, 1e-5, 8
    x = bf(rnd((T, (nq + nk) * hd + spare), 1))
    bias = rnd((nq + nk) * hd, 2, 0.5)
    rcfg = {"base": 300.0, "dims": rot}
    pos = np.array([0, 1, 5, 63, 64, 200, 3], dtype=np.int32)
    inv = torch.tensor(GP.rotary_frequencies(rcfg), dtype=torch.float32, device=DEV) if rot else None
    dst = torch.zeros((T, (nq + 2 * nk) * hd), dtype=dtype, device=DEV)
    ops.head_prep(dev(x, dtype), 0, nq, nk, nk * hd, hd, dst=dst, bias=dev(bias), norm_dim=hd, eps=eps, rot_dim=rot, inv_freq=inv,
                  interleaved=True, tok_pos=torch.tensor(pos, device=DEV), norm_last=True, plain_norm=True, values_are_keys=True)
    h = x[:, :(nq + nk) * hd].astype(np.float64) + bias
    want_v = h[:, nq * hd:]
    heads = h.reshape(T, nq + nk, hd)
    turned = np.stack([GP.rotate(heads[t:t + 1], rcfg, int(pos[t]))[0] for t in range(T)]) if rot else heads
    want = GP.rms_unit(turned, eps).reshape(T, -1)
    got = host(dst)
    tol = 3e-6 if dtype == torch.float32 else 0.02
    assert np.abs(got[:, :(nq + nk) * hd] - want).max() < tol * np.abs(want).max()
    assert np.abs(got[:, (nq + nk) * hd:] - want_v).max() < tol * np.abs(want_v).max()


# ---- the router with groups, experts without a gate ----------------------------------------------------------------

@pytest.mark.parametrize("experts,top,count,keep", [(16, 4, 4, 2), (6, 2, 6, 3), (8, 4, 2, 1), (12, 1, 3, 3), (9, 4, 3, 2),
                                                    (4, 4, 1, 1), (64, 6, 8, 2)])
def test_the_router_chooses_within_the_best_groups(experts, top, count, keep):
    from quicknn_b200.kernels import ops
    T, W = 40, 48
    h, wr = bf(rnd((T, W), 1)), bf(rnd((experts, W), 2, 0.6))
    corr = rnd(experts, 3, 0.3)
    if experts == 8:
        corr -= 3.0                                          # ranking values below zero: outside the groups is still lower
    w = {"router": wr.astype(np.float64), "correction": corr.astype(np.float64)}
    r = {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": count, "keep": keep}}
    chosen, weights = GP.route(h.astype(np.float64), w, "", r)
    for dtype in (torch.float32, torch.bfloat16):
        e, g = ops.moe_route(dev(h, dtype), dev(wr, dtype), top, "sigmoid", True, dev(corr), 2.5, groups=(count, keep))
        e, g = e.cpu().numpy().reshape(T, top), host(g).reshape(T, top)
        for t in range(T):
            assert e[t].tolist() == chosen[t].tolist(), f"row {t}"
            assert np.abs(g[t] - weights[t]).max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,count,keep,W,ff,shared,T", [(6, 2, 3, 2, 64, 32, 48, 21), (4, 4, 1, 1, 40, 24, None, 9),
                                                                   (8, 3, 4, 3, 128, 64, 64, 1500), (16, 1, 4, 1, 36, 20, 12, 70)])
def test_routed_experts_without_a_gate(dtype, experts, top, count, keep, W, ff, shared, T):
    """Few rows per expert (the tiles of decode steps) and many (the grouped tensor-core product of prompts)."""
    from quicknn_b200.parts import FEED_FORWARDS, PartSpec
    spec = PartSpec("routed_experts", {
        "hidden_size": W, "experts": experts, "top": top, "intermediate_size": ff, "gated": False, "activation": "relu2",
        "score": "sigmoid", "correction": True, "renormalize": True, "route_scale": 1.5, "groups": (count, keep),
        "weight_on": "output",
        "shared": None if shared is None else PartSpec("mlp", {"hidden_size": W, "intermediate_size": shared, "activation": "relu2"})})
    part = FEED_FORWARDS.get(spec.kind)(spec)
    w = {"router": bf(rnd((experts, W), 1, 2.0)), "correction": rnd(experts, 2, 0.1)}
    for e in range(experts):
        w[f"e{e}.up"], w[f"e{e}.down"] = bf(rnd((ff, W), 10 + e, 0.2)), bf(rnd((W, ff), 40 + e, 0.2))
    local = {"router": w["router"], "correction": w["correction"]}
    for e in range(experts):
        local[f"experts.{e}.up_proj"], local[f"experts.{e}.down_proj"] = w[f"e{e}.up"], w[f"e{e}.down"]
    if shared is not None:
        w["shared.up"], w["shared.down"] = bf(rnd((shared, W), 80, 0.2)), bf(rnd((W, shared), 81, 0.2))
        local["shared.up_proj"], local["shared.down_proj"] = w["shared.up"], w["shared.down"]
    part.load({k: dev(v, torch.float32 if k == "correction" else dtype) for k, v in local.items()}, dtype, DEV)
    h = bf(rnd((T, W), 5))
    mlp = {"router": {"experts": experts, "top": top, "scale": 1.5, "groups": {"count": count, "keep": keep}},
           "shared": None if shared is None else {"ff": shared}}
    want = GP.routed(h.astype(np.float64), f64(w), "", mlp)
    got = host(part.forward(dev(h, dtype), None))
    tol = 2e-5 if dtype == torch.float32 else 0.03
    bad = np.abs(got - want).max(axis=1) > tol * np.abs(want).max()
    assert bad.sum() <= (0 if dtype == torch.float32 else max(1, T // 30)), f"{int(bad.sum())} rows differ"


# ---- the sigmoid attention alone ---------------------------------------------------------------------------------

def attention_part(H, G, D, scale, chunk, rot, dtype, W=48, seed=0, kind="chunk", scaling=None):
    from quicknn_b200.config.tumudra import RotaryConfig
    from quicknn_b200.parts import MIXERS, PartSpec
    rcfg = {"base": 2000.0, "dims": rot}
    if scaling is not None:
        rcfg["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    spec = PartSpec("sigmoid_attention", {
        "hidden_size": W, "n_heads": H, "n_kv_heads": G, "head_dim": D, "scale": scale,
        "mask": {"kind": "causal", "size": 0} if chunk is None else {"kind": kind, "size": chunk}, "bias": True,
        "qk_norm": {"eps": 1e-5}, "head_bias": True, "talk": True, "out_gate": True, "values_from_keys": True,
        "position": RotaryConfig.parse(rcfg, "rot").part(D, "interleaved")})
    mixer = MIXERS.get(spec.kind)(spec)
    w = {"q": bf(rnd((H * D, W), seed + 1, 0.3)), "q.b": bf(rnd(H * D, seed + 2, 0.3)), "k": bf(rnd((G * D, W), seed + 3, 0.3)),
         "k.b": bf(rnd(G * D, seed + 4, 0.3)), "talk": bf(np.eye(H, dtype=np.float32) + rnd((H, H), seed + 5, 0.4)),
         "pb": bf(rnd(H, seed + 6, 0.5) - 1.0), "g": bf(rnd((H, W), seed + 7, 0.3)), "o": bf(rnd((W, H * D), seed + 8, 0.2))}
    names = {"q": "q_proj", "q.b": "q_bias", "k": "k_proj", "k.b": "k_bias", "talk": "talk", "pb": "head_bias",
             "g": "g_proj", "o": "o_proj"}
    mixer.load({names[k]: dev(v, dtype) for k, v in w.items()}, dtype, DEV)
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": scale, "rot": rcfg}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return mixer, w, m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,chunk,rot", [(4, 2, 16, 9, 8), (2, 2, 24, 1, 24), (6, 1, 64, 70, 64), (3, 3, 12, 64, 6),
                                             (8, 4, 64, 100, 32), (2, 1, 128, 130, 128), (1, 1, 8, 63, 0), (4, 4, 32, 65, 32),
                                             (5, 5, 40, None, 20)])
def test_sigmoid_attention_alone_and_a_chunk_one_position_off_would_show(dtype, H, G, D, chunk, rot):
    """Prompts of unequal lengths (one of a single token), then 70 tokens one by one, so that chunk edges, the page edge
    and the ring pass under decoded tokens; then a portion; then a slot that another sequence held."""
    from quicknn_b200.cache import KVCache
    mixer, w, m = attention_part(H, G, D, 0.9 / np.sqrt(D), chunk, rot, dtype, scaling=(4.0, 1.0, 4.0, 64) if rot >= 16 else None)
    W = 48
    cache = KVCache([mixer.cache_need()], [None], 2048, 4, 512, dtype, DEV)
    if chunk is not None:
        assert cache.line(0).ring == -(-chunk // 64) * 64
    w64 = f64(w)
    lens, extra = [200, 1, 67], 70
    xs = [bf(rnd((n + extra + 30, W), 30 + i)) for i, n in enumerate(lens)]
    ref = [GP.sigmoid_attention(x.astype(np.float64), w64, "", m, 1e-5) for x in xs]
    tol = (3e-5 if dtype == torch.float32 else 4e-2) * max(np.abs(r).max() for r in ref)
    if chunk is not None and dtype == torch.float32:         # the test can see an edge that is off by one
        for off in ((-1, 1) if chunk > 1 else (1,)):
            other = GP.sigmoid_attention(xs[0].astype(np.float64), w64, "", dict(m, mask={"size": chunk + off}), 1e-5)
            assert np.abs(other - ref[0]).max() > 20 * tol
    slots = [cache.allocate() for _ in lens]
    step = part_step(lens, [0, 0, 0], slots, "prefill", dtype, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)]), dtype), step, cache.line(0)))
    assert np.abs(y - np.concatenate([r[:n] for r, n in zip(ref, lens)])).max() < tol
    for t in range(extra):
        step = part_step([1, 1, 1], [n + t for n in lens], slots, "decode", dtype, cache, mixer)
        y = host(mixer.forward(dev(np.stack([x[n + t] for x, n in zip(xs, lens)]), dtype), step, cache.line(0)))
        want = np.stack([r[n + t] for r, n in zip(ref, lens)])
        assert np.abs(y - want).max() < tol, f"decoded token {t}"
    # a portion of 30 tokens onto the first sequence beside a single token of the third
    a, c = lens[0] + extra, lens[2] + extra
    step = part_step([30, 1], [a, c], [slots[0], slots[2]], "extend", dtype, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([xs[0][a:a + 30], xs[2][c:c + 1]]), dtype), step, cache.line(0)))
    assert np.abs(y - np.concatenate([ref[0][a:a + 30], ref[2][c:c + 1]])).max() < tol
    # the first sequence ends; a new one gets its slot and pages
    cache.free(slots[0])
    again = cache.allocate()
    x2 = bf(rnd((90, W), 77))
    step = part_step([90], [0], [again], "prefill", dtype, cache, mixer)
    y = host(mixer.forward(dev(x2, dtype), step, cache.line(0)))
    assert np.abs(y - GP.sigmoid_attention(x2.astype(np.float64), w64, "", m, 1e-5)).max() < tol


@pytest.mark.parametrize("chunk,far,where", [(88, 87, "decode"), (88, 88, "decode"), (40, 39, "prefill"), (40, 40, "prefill"),
                                             (None, 600, "decode"), (None, 600, "prefill"), (640, 600, "decode")])
def test_a_key_that_stands_out_just_inside_just_outside_and_far_back(chunk, far, where):
    """One token's key and value are made a hundred times larger than the others'; the row ``far`` positions later, at the
    last position of the chunk that the token opens (or the first of the next), shows whether it was seen.  In a prompt,
    and decoded after a prompt that ends just before the row (several ranges of keys where the context is long)."""
    from quicknn_b200.cache import KVCache
    H, G, D, W = 4, 2, 32, 48
    mixer, w, m = attention_part(H, G, D, 0.1, chunk, 16, torch.float32, seed=20)
    start = (chunk or 1) * 2                                 # the marked token opens a chunk
    n = start + far + 3
    x = bf(rnd((n, W), 5))
    x[start] *= 100.0
    ref = GP.sigmoid_attention(x.astype(np.float64), f64(w), "", m, 1e-5)
    blind = x.copy()
    blind[start] = 0.0
    seen = chunk is None or far < chunk
    row = start + far
    differs = np.abs(ref[row] - GP.sigmoid_attention(blind.astype(np.float64), f64(w), "", m, 1e-5)[row]).max()
    assert (differs > 0.5 * np.abs(ref[row]).max()) == seen
    cache = KVCache([mixer.cache_need()], [None], 4096, 2, 2048, torch.float32, DEV)
    slot = cache.allocate()
    tol = 3e-5 * np.abs(ref).max()
    if where == "prefill":
        step = part_step([n], [0], [slot], "prefill", torch.float32, cache, mixer)
        y = host(mixer.forward(dev(x), step, cache.line(0)))
        assert np.abs(y - ref).max() < tol
    else:
        step = part_step([row - 1], [0], [slot], "prefill", torch.float32, cache, mixer)
        mixer.forward(dev(x[:row - 1]), step, cache.line(0))
        for p in range(row - 1, n):
            step = part_step([1], [p], [slot], "decode", torch.float32, cache, mixer)
            step.tuning = {}                                  # the mixer's own number of key ranges
            y = host(mixer.forward(dev(x[p:p + 1]), step, cache.line(0)))
            assert np.abs(y[0] - ref[p]).max() < tol, f"position {p}"


@pytest.mark.parametrize("size", [1, 7, 64, 65, 100])
def test_a_sliding_window_instead_of_chunks(size):
    """The part's other mask: the last ``size`` positions.  A prompt, then 40 tokens one by one over the ring."""
    from quicknn_b200.cache import KVCache
    mixer, w, m = attention_part(4, 2, 16, 0.2, size, 8, torch.float32, seed=60, kind="window")
    cache = KVCache([mixer.cache_need()], [None], 1024, 2, 512, torch.float32, DEV)
    n, extra = 150, 40
    x = bf(rnd((n + extra, 48), 9))
    ref = GP.sigmoid_attention(x.astype(np.float64), f64(w), "", m, 1e-5, see=GP.window_visible(n + extra, size))
    tol = 3e-5 * np.abs(ref).max()
    slot = cache.allocate()
    step = part_step([n], [0], [slot], "prefill", torch.float32, cache, mixer)
    assert np.abs(host(mixer.forward(dev(x[:n]), step, cache.line(0))) - ref[:n]).max() < tol
    for p in range(n, n + extra):
        step = part_step([1], [p], [slot], "decode", torch.float32, cache, mixer)
        assert np.abs(host(mixer.forward(dev(x[p:p + 1]), step, cache.line(0)))[0] - ref[p]).max() < tol, f"position {p}"


def test_key_ranges_of_a_long_context_add_up():
    """Decode steps over 1500 cached tokens with 1, 3 and 16 ranges of keys per sequence give the same rows."""
    from quicknn_b200.cache import KVCache
    mixer, w, m = attention_part(4, 1, 64, 0.1, None, 64, torch.bfloat16, seed=40)
    cache = KVCache([mixer.cache_need()], [None], 4096, 2, 2048, torch.bfloat16, DEV)
    x = bf(rnd((1501, 48), 8))
    ref = GP.sigmoid_attention(x.astype(np.float64), f64(w), "", m, 1e-5)[1500]
    outs = []
    for splits in (1, 3, 16):
        slot = cache.allocate()
        step = part_step([1500], [0], [slot], "prefill", torch.bfloat16, cache, mixer)
        y = host(mixer.forward(dev(x[:1500], torch.bfloat16), step, cache.line(0)))
        if splits == 1:        # the prompt itself: on the tensor cores its far query tiles walk their keys in ranges too
            whole = GP.sigmoid_attention(x[:1500].astype(np.float64), f64(w), "", m, 1e-5)
            assert np.abs(y - whole).max() < 0.04 * np.abs(whole).max()
        step = part_step([1], [1500], [slot], "decode", torch.bfloat16, cache, mixer)
        step.tuning = {"decode_splits": splits}
        outs.append(host(mixer.forward(dev(x[1500:], torch.bfloat16), step, cache.line(0)))[0])
        cache.free(slot)
    for o in outs:
        assert np.abs(o - ref).max() < 0.04 * np.abs(ref).max()
    assert np.abs(outs[0] - outs[2]).max() < 0.01 * np.abs(ref).max()


# ---- the matrix memories alone --------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,heads,dim,vdim", [("lightning", 2, 16, 24), ("lightning", 1, 12, 40), ("lightning", 4, 32, 64),
                                                 ("lightning", 9, 8, 64),
                                                 ("hgrn2", 2, 16, 24), ("hgrn2", 1, 40, 12), ("hgrn2", 3, 4, 28), ("hgrn2", 2, 64, 32)])
def test_memories_alone_prompts_then_single_tokens_then_a_portion_then_a_reused_slot(dtype, kind, heads, dim, vdim):
    from quicknn_b200.cache import KVCache
    from quicknn_b200.parts import MIXERS, PartSpec
    W, eps = 40, 1e-5
    if kind == "lightning":
        decay = np.linspace(0.5, 0.999, heads).tolist()
        spec = PartSpec(kind, {"hidden_size": W, "n_heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "eps": eps})
        w = {"q": bf(rnd((heads * dim, W), 1, 0.3)), "k": bf(rnd((heads * dim, W), 2, 0.3)), "v": bf(rnd((heads * vdim, W), 3, 0.3)),
             "g": bf(rnd((heads * vdim, W), 4, 0.3)), "o": bf(rnd((W, heads * vdim), 5, 0.2)), "norm": bf(rnd(heads * vdim, 6, 0.2) + 1)}
        names = {"q": "q", "k": "k", "v": "v", "g": "gate", "o": "o", "norm": "norm"}
        m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
        plain = GP.lightning
    else:
        spec = PartSpec(kind, {"hidden_size": W, "n_heads": heads, "dim": dim, "vdim": vdim, "eps": eps})
        w = {"q": bf(rnd((heads * dim, W), 1, 0.3)), "f": bf(rnd((heads * dim, W), 2, 0.5)), "f.b": bf(rnd(heads * dim, 7) + 1.0),
             "lower": bf(np.linspace(0, 0.97, heads * dim)), "v": bf(rnd((heads * vdim, W), 3, 0.3)),
             "o": bf(rnd((W, heads * vdim), 5, 0.2)), "norm": bf(rnd(vdim, 6, 0.2) + 1)}
        names = {"q": "q", "f": "f", "f.b": "f_bias", "lower": "lower", "v": "v", "o": "o", "norm": "norm"}
        m = {"heads": heads, "dim": dim, "vdim": vdim}
        plain = GP.hgrn2
    mixer = MIXERS.get(kind)(spec)
    mixer.load({names[k]: dev(v, dtype) for k, v in w.items()}, dtype, DEV)
    cache = KVCache([None], [mixer.state_need()], 1024, 3, 512, dtype, DEV)
    lens, extra = [150, 1, 37], 8
    xs = [bf(rnd((n + extra + 20, W), 20 + i)) for i, n in enumerate(lens)]
    ref = [plain(x.astype(np.float64), f64(w), "", m, eps) for x in xs]
    tol = (3e-5 if dtype == torch.float32 else 5e-2) * max(np.abs(r).max() for r in ref)
    slots = [cache.allocate() for _ in lens][::-1]
    step = part_step(lens, [0, 0, 0], slots, "prefill", dtype, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)]), dtype), step, cache.line(0)))
    got, want = y, np.concatenate([r[:n] for r, n in zip(ref, lens)])
    # at a sequence's very first token the state has rank one and the norm keeps only a direction: bfloat16 may turn it
    rows = np.ones(len(want), dtype=bool)
    if dtype == torch.bfloat16:
        rows[[0, lens[0], lens[0] + lens[1]]] = False
    assert np.abs(got - want)[rows].max() < tol
    for t in range(extra):
        step = part_step([1, 1, 1], [n + t for n in lens], slots, "decode", dtype, cache, mixer)
        y = host(mixer.forward(dev(np.stack([x[n + t] for x, n in zip(xs, lens)]), dtype), step, cache.line(0)))
        assert np.abs(y - np.stack([r[n + t] for r, n in zip(ref, lens)])).max() < tol, f"decoded token {t}"
    a, c = lens[0] + extra, lens[2] + extra
    step = part_step([20, 2], [a, c], [slots[0], slots[2]], "extend", dtype, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([xs[0][a:a + 20], xs[2][c:c + 2]]), dtype), step, cache.line(0)))
    assert np.abs(y - np.concatenate([ref[0][a:a + 20], ref[2][c:c + 2]])).max() < tol
    cache.free(slots[0])
    again = cache.allocate()                                 # a state that another sequence left is zeroed
    x2 = bf(rnd((50, W), 77))
    step = part_step([50], [0], [again], "prefill", dtype, cache, mixer)
    y = host(mixer.forward(dev(x2, dtype), step, cache.line(0)))
    assert np.abs(y - plain(x2.astype(np.float64), f64(w), "", m, eps))[1:].max() < tol


def test_long_prompts_walk_the_memories_in_segments():
    from quicknn_b200.cache import KVCache
    from quicknn_b200.kernels import ops
    from quicknn_b200.parts import MIXERS, PartSpec
    W, heads, dim, vdim, eps = 32, 2, 16, 24, 1e-5
    spec = PartSpec("hgrn2", {"hidden_size": W, "n_heads": heads, "dim": dim, "vdim": vdim, "eps": eps})
    w = {"q": rnd((heads * dim, W), 1, 0.3), "f": rnd((heads * dim, W), 2, 0.5), "f.b": rnd(heads * dim, 7) + 2.0,
         "lower": np.linspace(0, 0.99, heads * dim).astype(np.float32), "v": rnd((heads * vdim, W), 3, 0.3),
         "o": rnd((W, heads * vdim), 5, 0.2), "norm": rnd(vdim, 6, 0.2) + 1}
    names = {"q": "q", "f": "f", "f.b": "f_bias", "lower": "lower", "v": "v", "o": "o", "norm": "norm"}
    mixer = MIXERS.get("hgrn2")(spec)
    mixer.load({names[k]: dev(v) for k, v in w.items()}, torch.float32, DEV)
    cache = KVCache([None], [mixer.state_need()], 4096, 3, 2048, torch.float32, DEV)
    lens = [700, 5, 300]
    assert max(lens) >= ops.GLA_SEGMENTS_FROM
    xs = [rnd((n + 600, W), 40 + i) for i, n in enumerate(lens)]
    ref = [GP.hgrn2(x.astype(np.float64), f64(w), "", {"heads": heads, "dim": dim, "vdim": vdim}, eps) for x in xs]
    slots = [cache.allocate() for _ in lens]
    step = part_step(lens, [0, 0, 0], slots, "prefill", torch.float32, cache, mixer)
    y = host(mixer.forward(dev(np.concatenate([x[:n] for x, n in zip(xs, lens)])), step, cache.line(0)))
    want = np.concatenate([r[:n] for r, n in zip(ref, lens)])
    assert np.abs(y - want).max() < 3e-5 * np.abs(want).max()
    step = part_step([600, 1], [700, 300], [slots[0], slots[2]], "extend", torch.float32, cache, mixer)   # onto a state that is not empty
    y = host(mixer.forward(dev(np.concatenate([xs[0][700:1300], xs[2][300:301]])), step, cache.line(0)))
    want = np.concatenate([ref[0][700:1300], ref[2][300:301]])
    assert np.abs(y - want).max() < 3e-5 * np.abs(want).max()


# ---- whole models ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("A", "bfloat16", False), ("B", "bfloat16", True),
                                              ("B", "float32", True), ("C", "float32", True), ("C", "bfloat16", True)])
def test_every_cutting_gives_the_plain_logits(guni, tmp_path, whole_model_tolerance, name, dtype, peaky):
    """Each request whole; its last 32 tokens one by one; batches of unequal lengths that shrink, one batch after
    another, so that slots, pages, rings and states are used again."""
    folder, plain = guni(name, dtype, peaky)
    routed_runs(CONFIGS[name][0])
    requests = prompts(name, LENGTHS_B if name == "B" else LENGTHS)
    ref = [plain.logits(t) for t in requests]
    replay = Replay(folder, dtype, tmp_path, max_tokens=576 if name == "B" else 384)
    try:
        worst = run_all_cuttings(replay, requests, ref, dtype)
    finally:
        replay.close()
    print(f"gunirax {name} {dtype} peaky={peaky}: largest error {worst:.3g}")


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_stream_after_every_executed_layer(guni, name):
    """A looped layer counts every time it runs; before a pass but the first the embedded rows have joined the stream."""
    from quicknn_b200.engine import Engine, Model
    folder, plain = guni(name, "float32", True)
    model = Model.from_folder(folder, "float32", DEV)
    engine = Engine(model, max_tokens=512)
    streams = []
    for blk in set(model.blocks):
        def wrap(resid, step, line, normed=None, next_norm=None, _inner=blk.forward):
            out = _inner(resid, step, line, normed=normed, next_norm=next_norm)
            streams.append(host(out[0] if isinstance(out, tuple) else out))
            return out
        blk.forward = wrap
    toks = prompts(name, [75])[0]
    engine.step([(engine.new_sequence(), toks)], [[len(toks) - 1]])
    want = plain.layers(toks)
    assert len(streams) == want.shape[0] == len(model.spec.schedule)
    for i, (got, ref) in enumerate(zip(streams, want)):
        assert np.abs(got - ref).max() < 3e-5 * np.abs(ref).max(), f"after executed layer {i}"


@pytest.mark.parametrize("name,dtype,peaky", [("A", "float32", True), ("B", "float32", True), ("B", "bfloat16", True),
                                              ("C", "float32", True)])
def test_prompts_in_portions_down_to_two_tokens(guni, tmp_path, name, dtype, peaky):
    """Steps that continue sequences by several tokens, beside requests that join or sit out."""
    folder, plain = guni(name, dtype, peaky)
    routed_runs(CONFIGS[name][0])
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
        step((0, a - 67 - 3), (2, 4), end=[2])   # a portion longer than the chunks
        step((0, 3), (1, b - 65), end=[0, 1])
        assert pos == [a, b, 45]
        got = replay.step([("again", requests[0], [a - 1])], end=["again"])      # what they held is free again
        ok, err, tol = near(got, ref[0][a - 1:a], dtype)
        assert ok, (err, tol)
    finally:
        replay.close()


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(guni, name):
    """More requests than slots, so that slots, rings and recurrent states are handed out again; decode steps run from
    CUDA graphs, one step ahead of the host; the tokens are the plain implementation's."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = guni(name, "float32", True)
    reqs = prompts(name, [5, 70, 1, 33, 12], seed=3)
    llm = LLM(folder, max_context=256, max_batch=2, dtype="float32")
    res = llm.generate(reqs, GenerationOptions.greedy(12), stop_ids=[])
    for r, p in zip(res, reqs):
        assert r.tokens == plain.greedy(p, 12), f"request {r.index}"
    llm16 = LLM(folder, max_context=256, max_batch=4, dtype="bfloat16")
    for r, p in zip(llm16.generate(reqs, GenerationOptions.greedy(6), stop_ids=[]), reqs):
        seq = list(p)
        for t in r.tokens:                      # bfloat16: every token is at least a near-best one of the plain logits
            row = plain.logits(seq)[-1]        # (the stack runs three times over; the rows' logits are of size 1)
            assert row[t] >= row.max() - 0.3 * max(1.0, np.abs(row).max())
            seq.append(t)


def test_long_decoding_keeps_states_rings_and_chunks(guni):
    """150 tokens generated one by one after a short prompt: chunks of 9 and of 1 position and the ring of a page pass
    over decoded tokens, the recurrent states of all passes of the loop are carried all the way."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, plain = guni("A", "float32", True)
    p = prompts("A", [3], seed=9)[0]
    llm = LLM(folder, max_context=256, max_batch=1, dtype="float32")
    got = llm.generate([p], GenerationOptions.greedy(150), stop_ids=[])[0].tokens
    seq = p + got
    ref = plain.logits(seq[:-1])
    for i, t in enumerate(got):                 # every generated token is the best one at its place
        row = ref[len(p) - 1 + i]
        assert row[t] >= row.max() - 1e-4 * max(1.0, np.abs(row).max()), f"token {i}"


def test_the_command_line_serves_the_design(guni, tmp_path):
    import subprocess
    import sys
    from conftest import ROOT

    def run(*argv):
        return subprocess.run([sys.executable, "-m", "quicknn_b200", *argv], cwd=ROOT, capture_output=True, text=True)
    folder, plain = guni("A", "float32", True)
    r = run("info", "--model", folder)
    assert r.returncode == 0, r.stderr
    info = json.loads(r.stdout)
    assert info["architecture"] == "Gunirax" and info["layers"] == len(GUNI_A["layers"])
    p = prompts("A", [9, 4], seed=5)
    r = run("generate", "--model", folder, "--prompt-ids", ";".join(",".join(map(str, q)) for q in p), "--max-new-tokens", "8",
            "--temperature", "0", "--dtype", "float32", "--max-context", "64", "--stop-ids", "")
    assert r.returncode == 0, r.stderr
    got = [json.loads(l) for l in r.stdout.splitlines() if l.strip()]
    assert [g["tokens"] for g in got] == [plain.greedy(q, 8) for q in p]
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(GUNI_C))
    out = tmp_path / "random_c"
    r = run("random", "--config", str(cfg), "--seed", "3", "--out", str(out), "--dtype", "bfloat16")
    assert r.returncode == 0, r.stderr
    ref = GP.PlainGunirax(str(out))
    toks = prompts("C", [21], seed=6)[0]
    replay = Replay(str(out), "float32", tmp_path / "logits", max_tokens=64)       # bfloat16 weights, widened exactly
    try:
        got = replay.step([("x", toks, range(len(toks)))], end=["x"])
    finally:
        replay.close()
    ok, err, tol = near(got, ref.logits(toks), "float32")
    assert ok, (err, tol)


def test_a_model_at_tensor_core_layer_sizes(tmp_path):
    """Head size 128, 16 heads on 4, widths in whole tiles, prompts of 600 tokens over chunks of 256: the products run
    on the tcgen05 kernels, the routed experts on the grouped product."""
    from quicknn_b200.engine import Engine, Model
    raw = dict(architecture="Gunirax", vocab=1024, width=512, embedding={"scale": 1.5}, norm={"eps": 1e-5},
               loop={"start": 0, "stop": 2, "times": 2}, initializer_range=0.04, layers=[
                   _par(_left(8, 2, 128, 0.06, 256, 64, 100000.0, (8.0, 1.0, 4.0, 512)), _right(4, 64, 128, (0.9, 0.95, 0.99, 0.999)),
                        _moe(256, 8, 2, 2.0, 4, 2, shared=256)),
                   _hgrn(4, 64, 128, _dense(1024))])
    CONFIGS["T"] = (raw, 11)
    routed_runs(raw)
    folder = make_folder(tmp_path, "T", "bfloat16", True)
    plain = GP.PlainGunirax(folder)
    model = Model.from_folder(folder, "bfloat16", DEV)
    engine = Engine(model, max_tokens=2048)
    reqs = prompts("T", [600, 300], seed=2)
    slots = [engine.new_sequence() for _ in reqs]
    rows = [[0, 255, 256, 257, 511, 512, 599], [0, 100, 299]]
    got = host(engine.step([(s, t) for s, t in zip(slots, reqs)], rows))
    want = np.concatenate([plain.logits(t)[r] for t, r in zip(reqs, rows)])
    ok, err, tol = near(got, want, "bfloat16")
    assert ok, (err, tol)
    nxt = [5, 9]
    got = host(engine.step([(s, [t]) for s, t in zip(slots, nxt)], [[0], [0]]))
    want = np.stack([plain.logits(t + [n])[-1] for t, n in zip(reqs, nxt)])
    ok, err, tol = near(got, want, "bfloat16")
    assert ok, (err, tol)


# ---- configurations drawn at random ---------------------------------------------------------------------------------

def random_config(seed):
    """Every size, the order of the layers, the loop and every constant drawn from a seed."""
    rng = np.random.default_rng(2000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]  # noqa: E731
    width = pick([48, 64, 96, 100, 160, 352])
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        kind = pick(["none", "dense", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = _dense(pick([32, 72, 128, 256]))
        else:
            count = pick([1, 2, 3, 4])
            per = pick([1, 2, 3, 4])
            keep = int(rng.integers(1, count + 1))
            top = int(rng.integers(1, min(4, keep * per) + 1))
            mlp = _moe(pick([16, 40, 64, 96]), count * per, top, pick([0.5, 1.0, 2.5]), count, keep, pick([None, 24, 32, 96]))
        if rng.random() < 0.65:
            kv = pick([1, 2, 3])
            dim = pick([8, 16, 24, 32, 64])
            dims = pick([0, dim // 2 // 2 * 2, dim])
            scaling = pick([None, (4.0, 1.0, 4.0, 64), (16.0, 0.5, 2.0, 256)])
            rh = int(rng.integers(1, 5))
            layers.append(_par(
                _left(kv * int(rng.integers(1, 4)), kv, dim, float(rng.uniform(0.05, 0.3)),
                      pick([None, 1, 3, 17, 63, 64, 65, 80, 100]), dims, pick([100.0, 10000.0, 500000.0]), scaling),
                _right(rh, pick([4, 8, 16, 32, 64]), pick([8, 16, 32, 64]), rng.uniform(0.3, 1.0, rh).tolist()), mlp))
        else:
            layers.append(_hgrn(int(rng.integers(1, 5)), pick([4, 8, 16, 32, 64, 128]), pick([8, 16, 32, 64]), mlp))
    n = len(layers)
    start = int(rng.integers(0, n + 1))
    stop = int(rng.integers(start, n + 1))
    raw = dict(architecture="Gunirax", vocab=int(rng.integers(100, 700)), width=width,
               embedding={"scale": float(pick([1.0, 0.5, 3.0]))}, norm={"eps": pick([1e-5, 1e-6])}, initializer_range=0.07,
               layers=layers)
    if rng.random() < 0.8:
        raw["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return raw


@pytest.mark.parametrize("seed", range(24))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Prompts of unequal lengths in one step, then tokens one by one, against the plain logits: float32 sharply for
    every configuration, bfloat16 for every other one."""
    from quicknn_b200.engine import Engine, Model
    raw = random_config(seed)
    name = f"R{seed}"
    CONFIGS[name] = (raw, 50 + seed)
    routed_runs(raw)
    lens, extra = [130, 7, 1, 70], 5
    reqs = prompts(name, [n + extra for n in lens], seed=seed)
    for dtype in (("float32", "bfloat16") if seed % 2 == 0 else ("float32",)):
        folder = make_folder(tmp_path, name, dtype, True)
        plain = GP.PlainGunirax(folder)
        ref = [plain.logits(t) for t in reqs]
        model = Model.from_folder(folder, dtype, DEV)
        engine = Engine(model, max_tokens=1024)
        slots = [engine.new_sequence() for _ in reqs]
        got = host(engine.step([(s, t[:n]) for s, t, n in zip(slots, reqs, lens)], [list(range(n)) for n in lens]))
        ok, err, tol = near(got, np.concatenate([r[:n] for r, n in zip(ref, lens)]), dtype)
        assert ok, f"{dtype} prompts: {err:.3g} > {tol:.3g}   {raw}"
        for k in range(extra):
            got = host(engine.step([(s, [t[n + k]]) for s, t, n in zip(slots, reqs, lens)], [[0]] * len(reqs)))
            ok, err, tol = near(got, np.stack([r[n + k] for r, n in zip(ref, lens)]), dtype)
            assert ok, f"{dtype} token {k}: {err:.3g} > {tol:.3g}   {raw}"
