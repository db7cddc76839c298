"""Where a step's time goes: CUDA events per step and per kind of part.

The reference can put timestamp queries around its command buffer
(src/backends/vulkan/QuickNN.Vulkan.Context.Implementation.inc:221-225) and reports time to the
first token, decode seconds and tokens per second for every reply
(src/models/QuickNN.Models.LLM.pas:851-857).  Here a ``StepProfiler`` wraps an engine for the
length of a ``with`` block: every step is bracketed by two events, and inside it every call of a
mixer, a feed-forward, a norm, the embedding, the output head and the sampler.  Steps run eagerly
meanwhile (events cannot be recorded inside a captured graph), so the per-step figures are those of
eager launches; the shares between the kinds of part are what the table is for.

    with StepProfiler(llm.engine) as prof:
        llm.generate(prompts, options)
    print(prof.table())

``StepProfiler(engine, nvtx=True)`` also opens an NVTX range of the part's kind around every call.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops
from ..parts.norm import RMSNorm
from ..sampling.sampler import Sampler

KINDS = ("embedding", "norms and residual", "mixer", "feed-forward", "head", "sampling")


class StepProfiler:
    def __init__(self, engine, nvtx: bool = False):
        self.engine = engine
        self.nvtx = nvtx                         # also an NVTX range around every call of a part, for a timeline tool
        self._undo: List[Tuple[object, str, object]] = []
        self._open: List[list] = []            # the calls that are running: [kind, start, stop, time of the calls inside]
        self._calls: List[list] = []
        self._steps: List[Tuple[str, int, int, torch.cuda.Event, torch.cuda.Event]] = []
        self._graphs: Optional[bool] = None

    # ---- wrapping ------------------------------------------------------------------------------
    def _timed(self, kind: str, fn):
        def call(*a, **kw):
            rec = [kind, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), []]
            if self._open:
                self._open[-1][3].append(rec)
            else:
                self._calls.append(rec)
            self._open.append(rec)
            if self.nvtx:
                torch.cuda.nvtx.range_push(kind)
            rec[1].record()
            try:
                return fn(*a, **kw)
            finally:
                rec[2].record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
                self._open.pop()
        return call

    def _patch(self, owner, name: str, kind: str) -> None:
        old = getattr(owner, name)
        self._undo.append((owner, name, owner.__dict__.get(name, _MISSING) if not isinstance(owner, type) else old))
        setattr(owner, name, self._timed(kind, old))

    def __enter__(self) -> "StepProfiler":
        eng, model = self.engine, self.engine.model
        self._graphs, eng.use_graphs = eng.use_graphs, False
        for blk in model.blocks:
            self._patch(blk.mixer, "forward", "mixer")
            if blk.ff is not None:
                self._patch(blk.ff, "forward", "feed-forward")
        self._patch(RMSNorm, "__call__", "norms and residual")
        self._patch(RMSNorm, "add_to", "norms and residual")
        self._patch(ops, "add_", "norms and residual")
        self._patch(ops, "add_scaled_rmsnorm", "norms and residual")
        self._patch(ops, "embed", "embedding")
        self._patch(ops, "embed_rmsnorm", "embedding")
        self._patch(model, "logits_of_rows", "head")
        self._patch(Sampler, "__call__", "sampling")
        self._patch(Sampler, "head", "sampling")
        for name in ("step", "decode"):
            old = getattr(eng, name)
            self._undo.append((eng, name, _MISSING))

            def stepped(*a, _old=old, _name=name, **kw):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                try:
                    return _old(*a, **kw)
                finally:
                    e1.record()
                    entries = a[0]
                    rows = len(entries)
                    toks = rows if _name == "decode" else sum(len(t) for _, t in entries)
                    mode = "decode" if toks == rows and _name == "decode" else ("prompt" if toks > rows else "single")
                    self._steps.append((mode, rows, toks, e0, e1))
            setattr(eng, name, stepped)
        return self

    def __exit__(self, *exc) -> None:
        for owner, name, old in reversed(self._undo):
            if old is _MISSING:
                try:
                    delattr(owner, name)
                except AttributeError:
                    pass
            else:
                setattr(owner, name, old)
        self._undo.clear()
        self.engine.use_graphs = self._graphs
        torch.cuda.synchronize(self.engine.device)

    # ---- results -------------------------------------------------------------------------------
    def by_kind(self) -> Dict[str, float]:
        """Milliseconds per kind of part, each call counted without the calls inside it."""
        out = {k: 0.0 for k in KINDS}

        def walk(rec) -> float:
            total = rec[1].elapsed_time(rec[2])
            inner = sum(walk(r) for r in rec[3])
            out[rec[0]] = out.get(rec[0], 0.0) + max(0.0, total - inner)
            return total
        for rec in self._calls:
            walk(rec)
        return out

    def steps(self) -> Dict[str, Tuple[int, int, float]]:
        """mode -> (steps, tokens, milliseconds)."""
        out: Dict[str, List[float]] = {}
        for mode, rows, toks, e0, e1 in self._steps:
            s = out.setdefault(mode, [0, 0, 0.0])
            s[0] += 1
            s[1] += toks
            s[2] += e0.elapsed_time(e1)
        return {k: (int(v[0]), int(v[1]), float(v[2])) for k, v in out.items()}

    def table(self) -> str:
        torch.cuda.synchronize(self.engine.device)
        lines = ["steps (launched eagerly while profiling):"]
        for mode, (n, toks, ms) in sorted(self.steps().items()):
            lines.append(f"  {mode:8s} {n:6d} steps {toks:9d} tokens {ms:10.3f} ms {toks / max(ms, 1e-9) * 1e3:12.1f} tokens/s")
        kinds = self.by_kind()
        total = sum(kinds.values()) or 1.0
        lines.append("time on the device by kind of part:")
        for k in KINDS:
            lines.append(f"  {k:20s} {kinds[k]:10.3f} ms {100.0 * kinds[k] / total:6.1f} %")
        return "\n".join(lines)


class _Missing:
    pass


_MISSING = _Missing()


# ---- time and roofline by kernel wrapper ------------------------------------------------------------------

def _nbytes(t) -> int:
    return t.numel() * t.element_size() if isinstance(t, torch.Tensor) else 0


def _tensors(xs):
    for x in xs:
        if isinstance(x, torch.Tensor):
            yield x
        elif isinstance(x, (tuple, list)):
            yield from _tensors(x)


class OpTimer:
    """Brackets every call of the kernel wrappers in ``kernels.ops`` with CUDA events while steps run eagerly, and
    sets each wrapper's time against the least time its work could take: the bytes it has to move at ``hbm_gbs``
    or its floating-point operations at ``tflops``, whichever is longer.  Bytes are those of the tensors that go
    in and come out, except where a wrapper reads a part of its arguments only (decode attention reads the live
    keys, not the pool; routed experts read the chosen experts' matrices); operations are counted for products,
    attention, the linear-attention scan and the experts.  ``context`` is the number of cached positions that a
    decode step's attention walks (the timer cannot see lengths that live on the device); prompts are taken to
    be one sequence per step.

        with OpTimer(engine, hbm_gbs=6500, tflops=1600, context=4096) as t:
            engine.step(...)
        for row in t.rows(): print(row)
    """

    SKIP = {"status_words", "finite_flag", "raise_on_status", "check_gemm_status", "wait_status_message", "dt_code",
            "attention_refusal", "linear_refusal", "sample_scratch_bytes", "head_candidates", "head_argmax_fusable",
            "qkv_rope_cache_fusable", "cache_append", "gemm_tcgen05", "gemm_skinny_tcgen05", "activation_"}

    def __init__(self, engine, hbm_gbs: float, tflops: float, context: int = 0):
        self.engine, self.hbm, self.tflops, self.context = engine, hbm_gbs * 1e9, tflops * 1e12, context
        self._undo: List[Tuple[str, object]] = []
        self._recs: List[tuple] = []
        self._depth = 0
        self._graphs: Optional[bool] = None

    def _cost(self, name: str, a, kw, out) -> Tuple[float, float]:
        """(bytes, floating-point operations) of one call."""
        byts = float(sum(_nbytes(t) for t in _tensors(a)) + sum(_nbytes(t) for t in _tensors(kw.values()))
                     + sum(_nbytes(t) for t in _tensors([out])))
        flops = 0.0
        if name == "linear":
            x, w = a[0], a[1]
            flops = 2.0 * x.shape[0] * w.shape[0] * w.shape[1]
        elif name == "small_linear_f32":
            flops = 2.0 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
        elif name == "attn_prefill":
            qkv, nq, nkv, hd, window = a[0], a[1], a[2], a[3], a[8]
            T = qkv.shape[0]
            keys = sum(min(p + 1, window) if window else p + 1 for p in range(T))
            flops = 4.0 * nq * hd * keys
        elif name == "attn_decode":
            qkv, nq, nkv, hd, k_pool, v_pool, window = a[0], a[1], a[2], a[3], a[4], a[5], a[13]
            seen = min(self.context, window) if window else self.context
            pools = 1 if v_pool.data_ptr() == k_pool.data_ptr() else 2
            byts = float(qkv.shape[0] * seen * nkv * hd * k_pool.element_size() * pools + _nbytes(qkv) + _nbytes(out))
            flops = 4.0 * qkv.shape[0] * nq * hd * seen
        elif name == "sigmoid_attention":
            qkv, nq, nkv, hd = a[0], a[1], a[2], a[3]
            kind, size, T = kw.get("mask", "causal"), int(kw.get("mask_size") or 0), qkv.shape[0]

            def seen(p):                         # keys that position p sees
                return p + 1 if kind == "causal" else (min(p + 1, size) if kind == "window" else p % size + 1)
            if kw.get("own_rows", True):
                flops = 4.0 * nq * hd * sum(seen(p) for p in range(T))
            else:
                keys = seen(max(0, self.context - 1))
                byts = float(T * keys * nkv * hd * qkv.element_size() * 2 + _nbytes(qkv) + _nbytes(out))
                flops = 4.0 * T * nq * hd * keys
        elif name == "gla_scan":
            proj, n_seqs, H, dim, vdim = a[0], a[10], a[11], a[12], a[13]
            T = proj.shape[0]
            flops = 4.0 * T * H * dim * vdim
            byts = float(T * (2 * H * dim + H * vdim) * proj.element_size() + T * H * dim * 4 + T * H * vdim * 4
                         + 2 * n_seqs * H * dim * vdim * 4)
        elif name == "memory_scan":
            proj, normaliser, n_seqs, H, dim, vdim = a[0], a[9], a[14], a[15], a[16], a[17]
            T, vs = proj.shape[0], vdim + (1 if normaliser else 0)
            flops = 4.0 * T * H * dim * vs
            byts = float(T * (2 * H * dim + H * vdim) * proj.element_size() + T * H * vs * 4 + 2 * n_seqs * H * dim * vs * 4)
        elif name == "attn_prefill_paged":
            qkv, nq, nkv, hd, window = a[0], a[1], a[2], a[3], a[13]
            T = qkv.shape[0]
            keys = sum(min(p + 1, window) if window else p + 1 for p in range(T))
            flops = 4.0 * nq * hd * keys
            byts = float(T * nq * hd * qkv.element_size() * 2 + 2 * T * nkv * hd * qkv.element_size())
        elif name == "head_prep":
            src, nq, nk, nv, hd = a[0], a[2], a[3], a[4], a[5]
            dst = kw.get("dst")
            width = (nq + nk) * hd + nv
            byts = float(src.shape[0] * width * (src.element_size() + (dst.element_size() if dst is not None else src.element_size())))
        elif name == "moe_experts":
            x, top, wgu, wd = a[0], a[3], a[4], a[5]
            T, W = x.shape
            E, ff2, _ = wgu.shape
            used = min(E, T * top)
            rows = ff2 + (ff2 // 2 if kw.get("gated", True) else ff2)        # rows of an expert's matrices
            flops = 2.0 * T * top * rows * W
            byts = float(used * rows * W * wgu.element_size() + _nbytes(x) + _nbytes(out))
        elif name in ("rope_cache_write",):
            byts = float(2 * _nbytes(a[0]))
        elif name.startswith("embed"):               # the rows that are looked up, not the table
            byts = float(2 * sum(_nbytes(t) for t in _tensors([out])))
        return byts, flops

    def _timed(self, name: str, fn):
        def call(*a, **kw):
            if self._depth:                      # a wrapper called from inside another: the outer one is counted
                return fn(*a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._depth += 1
            e0.record()
            try:
                out = fn(*a, **kw)
            finally:
                e1.record()
                self._depth -= 1
            self._recs.append((name, e0, e1) + self._cost(name, a, kw, out))
            return out
        return call

    def __enter__(self) -> "OpTimer":
        self._graphs, self.engine.use_graphs = self.engine.use_graphs, False
        for name, fn in list(vars(ops).items()):
            if callable(fn) and not name.startswith("_") and getattr(fn, "__module__", "") == ops.__name__ \
                    and not isinstance(fn, type) and name not in self.SKIP:
                self._undo.append((name, fn))
                setattr(ops, name, self._timed(name, fn))
        return self

    def __exit__(self, *exc) -> None:
        for name, fn in self._undo:
            setattr(ops, name, fn)
        self._undo.clear()
        self.engine.use_graphs = self._graphs
        torch.cuda.synchronize(self.engine.device)

    def rows(self) -> List[Dict[str, object]]:
        """One record per wrapper, the costliest first: calls, milliseconds, the least milliseconds its bytes and
        operations allow, and the quotient (1.0 = at the roofline)."""
        torch.cuda.synchronize(self.engine.device)
        agg: Dict[str, List[float]] = {}
        for name, e0, e1, byts, flops in self._recs:
            r = agg.setdefault(name, [0, 0.0, 0.0, 0.0, 0.0])
            r[0] += 1
            r[1] += e0.elapsed_time(e1)
            r[2] += max(byts / self.hbm, flops / self.tflops) * 1e3
            r[3] += byts
            r[4] += flops
        out = [{"op": k, "calls": int(v[0]), "ms": round(v[1], 4), "least_ms": round(v[2], 4),
                "of_roofline": round(v[2] / v[1], 4) if v[1] > 0 else None, "gb": round(v[3] / 1e9, 4),
                "gflop": round(v[4] / 1e9, 2)} for k, v in agg.items()]
        return sorted(out, key=lambda r: -r["ms"])
