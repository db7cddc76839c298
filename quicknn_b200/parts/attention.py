"""The attention mixer: grouped-query attention over the paged cache, with the window,
the softcap and the scale as parameters.

Order of operations as in the reference's layer body
(src/models/QuickNN.Models.Gemma2.pas:167-180): Q, K, V projections; rotation of Q and K;
append K, V to the cache; attention with scale 1/sqrt(query_pre_attn_scalar), softcap
and window; output projection.  The three projections are one product against the
stacked matrix; rotation and append belong to the position part (one kernel, or, for the
few rows of a decode step, the epilogue of that product).

Options beyond that (all off unless the spec gives them):

* ``v_head_dim``: a value size that differs from the key size ``head_dim``.  Heads are carried at one internal size,
  the larger of the two rounded up to a whole 16-byte piece, with zero rows in the stacked matrix behind the shorter
  kind (zero query/key columns add nothing to a score, zero value columns meet zero columns of the output matrix), so
  every attention kernel of the library serves them; the cache line has the internal size.
* ``bias``: biases on the q, k, v and o products (``q_bias`` ... ``o_bias``).
* ``qk_norm`` = {"eps": e}: an RMS norm over ``head_dim`` per query head and key head with the weights ``q_norm`` /
  ``k_norm`` (shared by the heads), before the rotation.
  With ``"over": "projection"`` it is one norm over the whole query projection (all heads together) and one over the
  whole key projection, with weights of those sizes.
* ``distance_slopes``: one number per query head; ``slope * (i - j)`` is subtracted from the score of query position i and
  key position j (a bias that grows with the distance, in float32 inside the attention kernels).
* ``out_gate``: the concatenated heads are multiplied, element by element, by sigmoid(``g_proj`` x) before the output
  product.
* ``shared_kv``: the layer has no keys and values of its own; its schedule entry reads the cache line that another
  layer writes (whose head counts, sizes and rotation are the same), with its own queries.

Decode attention cuts each sequence's keys into ranges that run as separate blocks and are
merged afterwards; how many ranges, and the scratch that the partial results need, are
decided here (``tuning["decode_splits"]`` fixes the number).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheNeed, HeadPrep, HeadShape, Mixer
from .linear import project, stack_rows
from .spec import PartSpec


BLOCK_COST = 64.0        # a decode-attention block's fixed cost, in keys of its walk
MERGE_COST = 100.0       # the kernel that merges more than four ranges, in the same unit


@MIXERS.register("attention")
class AttentionMixer(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.softcap = p.get("softcap")
        self.window = p.get("window")
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_kv} kv heads do not divide {self.n_heads} heads")
        # key size and value size as the checkpoint has them; `head_dim` from here on is the size heads are carried at
        self.key_dim = self.head_dim
        self.value_dim = int(p.get("v_head_dim") or self.head_dim)
        self.has_bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        self.shared_kv = bool(p.get("shared_kv", False))
        self.norm_whole = bool(self.qk_norm) and self.qk_norm.get("over", "head") == "projection"
        self.out_gate = bool(p.get("out_gate", False))
        self._slope_values = None if p.get("distance_slopes") is None else tuple(float(v) for v in p["distance_slopes"])
        if self._slope_values is not None and len(self._slope_values) != self.n_heads:
            raise ValueError(f"{len(self._slope_values)} distance slopes for {self.n_heads} heads")
        self.slopes: Optional[torch.Tensor] = None
        self.w_out_gate: Optional[torch.Tensor] = None
        if p.get("v_head_dim") and (self.value_dim != self.key_dim or self.key_dim % 8):
            self.head_dim = (max(self.key_dim, self.value_dim) + 7) // 8 * 8
        self.heads = HeadShape(self.n_heads, 0 if self.shared_kv else self.n_kv, self.head_dim)
        pos: PartSpec = p["position"]
        if self.head_dim != self.key_dim and "head_dim" in pos.params:
            pos = PartSpec(pos.kind, dict(pos.params, head_dim=self.head_dim,
                                          rotary_dim=pos.get("rotary_dim", self.key_dim)))
        self.position = POSITIONS.get(pos.kind)(pos)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.out_bias: Optional[torch.Tensor] = None
        # a block that adds the output's bias in its own kernel (with the norm and the add that follow) sets this
        self.defer_out_bias = False
        self.prep: Optional[HeadPrep] = None
        self._resident = 148

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        H, nq, nkv, hd = int(p["hidden_size"]), int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        vd = int(p.get("v_head_dim") or hd)
        M, B, S = cls.PARAM_ROLE_MATRIX, cls.PARAM_ROLE_NORM, cls.PARAM_ROLE_SCALE
        shared = bool(p.get("shared_kv", False))
        out = {"q_proj": ((nq * hd, H), M), "o_proj": ((H, nq * vd), M)}
        if not shared:
            out.update({"k_proj": ((nkv * hd, H), M), "v_proj": ((nkv * vd, H), M)})
        if p.get("bias", False):
            out.update({"q_bias": ((nq * hd,), B), "o_bias": ((H,), B)})
            if not shared:
                out.update({"k_bias": ((nkv * hd,), B), "v_bias": ((nkv * vd,), B)})
        if p.get("qk_norm"):
            whole = p["qk_norm"].get("over", "head") == "projection"
            out["q_norm"] = ((nq * hd if whole else hd,), S)
            if not shared:
                out["k_norm"] = ((nkv * hd if whole else hd,), S)
        if p.get("out_gate", False):
            out["g_proj"] = ((nq * vd, H), M)
        return out

    def _carried(self, t: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """Rows (or elements) of ``heads`` heads of ``size`` each, laid out at the carried head size with zeros behind."""
        if size == self.head_dim:
            return t
        out = torch.zeros((heads, self.head_dim) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        out[:, :size] = t.reshape((heads, size) + tuple(t.shape[1:]))
        return out.reshape((heads * self.head_dim,) + tuple(t.shape[1:]))

    def load(self, tensors, compute_dtype, device) -> None:
        kd, vd, D = self.key_dim, self.value_dim, self.head_dim
        parts = [self._carried(tensors["q_proj"], self.n_heads, kd)]
        biases = [self._carried(tensors["q_bias"], self.n_heads, kd)] if self.has_bias else []
        if not self.shared_kv:
            parts += [self._carried(tensors["k_proj"], self.n_kv, kd), self._carried(tensors["v_proj"], self.n_kv, vd)]
            if self.has_bias:
                biases += [self._carried(tensors["k_bias"], self.n_kv, kd), self._carried(tensors["v_bias"], self.n_kv, vd)]
        self.w_qkv = stack_rows(parts)
        self.w_qkvg = None
        w_o = tensors["o_proj"]
        if vd != D:                                          # zero columns where the carried values are zero
            wide = torch.zeros((w_o.shape[0], self.n_heads, D), dtype=w_o.dtype, device=w_o.device)
            wide[:, :, :vd] = w_o.reshape(w_o.shape[0], self.n_heads, vd)
            w_o = wide.reshape(w_o.shape[0], self.n_heads * D)
        self.w_o = w_o.contiguous()
        self.out_bias = tensors["o_bias"].contiguous() if self.has_bias else None
        if self.out_gate:                                    # zero rows where the carried values are zero
            self.w_out_gate = self._carried(tensors["g_proj"], self.n_heads, vd).contiguous()
            if self.w_out_gate.dtype == self.w_qkv.dtype:
                # one matrix q | k | v | g, of which the two above are the row ranges: a decode step forms all four in one
                # product (its kernels take rows wider than what they read), a prompt keeps two, since the prompt
                # attention wants its rows packed
                self.w_qkvg = stack_rows([self.w_qkv, self.w_out_gate])
                n = self.w_qkv.shape[0]
                self.w_qkv, self.w_out_gate = self.w_qkvg[:n], self.w_qkvg[n:]
        if self._slope_values is not None:
            self.slopes = torch.tensor(self._slope_values, dtype=torch.float32, device=device)
        if self.has_bias or self.qk_norm:
            self.prep = HeadPrep(
                bias=torch.cat([b.to(torch.float32) for b in biases]).contiguous() if biases else None,
                q_norm=tensors["q_norm"].contiguous() if self.qk_norm else None,
                k_norm=tensors["k_norm"].contiguous() if self.qk_norm and not self.shared_kv else None,
                norm_dim=kd if self.qk_norm else 0, eps=float(self.qk_norm["eps"]) if self.qk_norm else 0.0,
                whole=self.norm_whole)
        self.position.prepare(device)
        # sizes that the kernels do not take are refused here, when the model is built, not at its first step
        why = (ops.attention_refusal(compute_dtype, self.n_heads, self.n_kv, self.head_dim)
               or ops.linear_refusal(self.w_qkv.dtype, self.hidden)
               or ops.linear_refusal(self.w_o.dtype, self.n_heads * self.head_dim))
        if why:
            raise ValueError(f"attention mixer: {why}")
        # blocks of the decode attention kernel that the device holds at once: its shared memory is
        # 384 bytes per element of a head, so two fit on an SM at head size 256, four at 128, eight at 64
        dev = torch.device(device)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 148
        self._resident = sms * max(1, min(8, 512 // max(1, self.head_dim)))

    def weight_bytes(self) -> int:
        ws = [self.w_qkv, self.w_o, self.out_bias, self.w_out_gate]
        if self.prep is not None:
            ws += [self.prep.bias, self.prep.q_norm, self.prep.k_norm]
        return sum(w.numel() * w.element_size() for w in ws if w is not None)

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(self.n_kv, self.head_dim, self.window)

    def decode_splits(self, step) -> int:
        """Key ranges per sequence in a decode step: a fixed number when the engine's owner gave one, else the
        number with the shortest estimated time for the step's length classes (``step.longest``, ``step.spread``).

        A sequence's keys are cut into equal ranges, a block per (range, kv head, sequence).  While all blocks
        fit the device at once the step takes as long as the longest sequence's range.  With more blocks than
        that they run in turns: blocks of one length (sequences of nearly equal lengths) in whole rounds, each as
        long as a block; blocks of unequal lengths fill the device evenly, and the time is the work of all blocks
        spread over the device plus about half a block at the end.  A block costs about as much as 64 keys before
        its first key, and more than four ranges are merged by a kernel of its own, which costs about as much as a
        hundred.  Measured at head size 256, context 8192, equal lengths, 6 layers, ms per step by ranges: batch 24:
        2: 1.32, 3: 1.08, 4: 1.34, 5: 1.20, 6: 1.11, 8: 1.18 (one round of 288 blocks, then 2, 2, 2 and 3 rounds);
        batch 28: 2: 1.34, 3: 1.60, 5: 1.23, 6: 1.39; batch 12: 4: 0.91, 5: 0.85, 6: 0.81, 8: 0.94; batch 64 one
        range 9.48 ms (26 layers) against two 9.69 and eight 8.42; batch 64 with prompts of 512 to 2048 tokens one
        range 4.20 ms, four 4.03, six 3.90, nine 4.12 (the longest sequence no longer sets the pace).  Results
        differ between these choices by rounding only: ranges are summed in a fixed order."""
        fixed = step.tuning.get("decode_splits")
        if fixed:
            return int(fixed)
        tiles = max(1, step.n_seqs * self.n_kv)
        longest = step.longest or step.max_seq
        if self.window:
            longest = min(longest, self.window)
        most = max(1, min(64, longest // 32))
        mean = longest / (step.spread or 1.0)
        best, best_time = 1, float("inf")
        equal = (step.spread or 1.0) <= 1.0
        for s in range(1, most + 1):                 # times in keys of one block's walk
            if s * tiles <= self._resident:
                t = longest / s + BLOCK_COST
            elif equal:                              # blocks of one length run in rounds
                t = -(-s * tiles // self._resident) * (longest / s + BLOCK_COST)
            else:
                t = tiles * (mean + s * BLOCK_COST) / self._resident + longest / (2 * s)
            if s > 4:
                t += MERGE_COST
            if t < best_time * 0.999:
                best, best_time = s, t
        return best

    def schedule(self, step) -> tuple:
        return (self.decode_splits(step),) if step.mode == "decode" else ()

    def scratch_need(self, step) -> int:
        """Partial (maximum, sum, output) of every key range: float32, [rows, heads, ranges, head_dim + 2]."""
        if step.mode != "decode":
            return 0
        return step.n_seqs * self.n_heads * self.decode_splits(step) * (self.head_dim + 2) * 4

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        h = self.heads
        extend = step.mode == "extend"
        fusable = not extend and self.prep is None and not self.shared_kv
        qkv = self.position.project_and_place(x, self.w_qkv, h, step, line) if fusable else None
        gate_col = 0
        if qkv is None:
            if self.w_qkvg is not None and step.mode == "decode":
                qkv, gate_col = project(x, self.w_qkvg), self.w_qkv.shape[0]
            else:
                qkv = project(x, self.w_qkv)
            if self.prep is None:
                self.position.place(qkv, h, step, line, append=not extend)
            else:
                self.position.place(qkv, h, step, line, append=not extend, prep=self.prep)
        if line.has_readers and line.writes and not self.shared_kv and step.mode != "decode":
            step.shared_rows[line.index] = (qkv, h)          # for the layers that read this line later in the step
        a = self.attend(qkv, step, line)
        if gate_col:
            a = ops.sigmoid_gate_(a, qkv, gate_col)
        elif self.out_gate:
            a = ops.sigmoid_gate_(a, project(x, self.w_out_gate))
        y = project(a, self.w_o)
        return y if (self.out_bias is None or self.defer_out_bias) else ops.add_bias_(y, self.out_bias)

    def _attend_rows_of(self, left, q: torch.Tensor, step, line) -> torch.Tensor:
        """Attention of the query rows ``q`` (the first columns of its rows) over the keys and values in the packed rows
        ``left`` = (rows, head shape) that the writer of the cache line left for this step: whole prompts over those
        rows alone; a step that continues sequences over the cache as earlier steps left it and those rows from there
        on (the writer appends them when the step's last layer is through)."""
        rows, shape = left
        D, nkv = self.head_dim, self.n_kv
        if shape.head_dim != D or shape.n_kv_heads != nkv or rows.shape[0] != q.shape[0] or rows.dtype != q.dtype:
            raise ValueError("the rows that the cache line's writer left do not fit this layer's heads")
        packed = torch.empty((q.shape[0], (self.n_heads + 2 * nkv) * D), dtype=q.dtype, device=q.device)
        ops.copy_col_range(q, 0, self.n_heads * D, packed, 0)
        ops.copy_col_range(rows, shape.n_heads * D, 2 * nkv * D, packed, self.n_heads * D)
        if step.mode == "extend":
            return ops.attn_extend(packed, self.n_heads, nkv, D, line.k, line.v, line.page_table, line.page_size,
                                   line.ring, step.tok_pos, step.tok_row0, step.tok_slot, self.scale, self.softcap,
                                   self.window, whole=getattr(step, "whole", None), slopes=self.slopes)
        return ops.attn_prefill(packed, self.n_heads, nkv, D, step.tok_pos, step.tok_row0, self.scale, self.softcap,
                                self.window, step.seq_row0, step.seq_len, step.max_q_len, slopes=self.slopes)

    def attend(self, qkv: torch.Tensor, step, line) -> torch.Tensor:
        """Attention of the packed q|k|v rows of a step, by the step's mode.  In prefill and decode the keys and
        values are in the cache line already; a step that continues sequences by several rows appends them
        here, after the attention.  Returns [rows, heads * head_dim]."""
        h = self.heads
        extend = step.mode == "extend"
        if extend and line.writes and not self.shared_kv:
            # cached keys from before this step, this step's own rows from there on; the append comes last,
            # so that the first rows still find the ring cells that the last rows overwrite
            a = ops.attn_extend(qkv, h.n_heads, h.n_kv_heads, h.head_dim, line.k, line.v, line.page_table,
                                line.page_size, line.ring, step.tok_pos, step.tok_row0, step.tok_slot, self.scale,
                                self.softcap, self.window, whole=getattr(step, "whole", None), slopes=self.slopes)
            append = lambda: ops.cache_append(qkv, h.n_heads, h.n_kv_heads, h.head_dim, step.tok_pos, step.tok_slot, line)  # noqa: E731
            if line.has_readers and hasattr(step, "after_layers"):
                step.after_layers.append(append)             # the line's readers come first: see _attend_rows_of
            else:
                append()
        elif step.mode != "decode" and (not line.writes or self.shared_kv):
            # the keys of this line were written by another layer earlier in this step; in a ring the last
            # rows of the step have by then overwritten cells: whole prompts may fill the ring, a step that
            # continues a sequence may bring only as many rows as the ring has cells beyond the window
            left = step.shared_rows.get(line.index)
            if left is not None and (extend or qkv.shape[1] == self.n_heads * self.head_dim):
                # this step's keys and values are the rows that the line's writer left, so the layer attends over
                # packed rows of its own queries beside them, like the writer itself (a prompt longer than a ring, or
                # a portion longer than the ring's spare cells, is no matter then)
                return self._attend_rows_of(left, qkv, step, line)
            room = line.ring - ((self.window or line.ring) - 1 if extend else 0)
            if line.ring and step.max_q_len > room:
                raise ValueError(f"a step of {step.max_q_len} tokens overruns the ring of {line.ring} "
                                 f"positions that this layer reads from another layer's cache line")
            a = None
            whole = getattr(step, "whole", None) if extend else None
            if qkv.shape[1] == self.n_heads * self.head_dim and step.seq_row0 is not None and (whole is not None or not extend):
                # queries only, every key in the cache: whole sequences for the tensor-core prompt kernel
                a = ops.attn_shared_tensor_core(qkv, self.n_heads, self.n_kv, self.head_dim, line.k, line.v,
                                                line.page_table, line.page_size, line.ring, step.slots, step.seq_row0,
                                                step.seq_len, self.scale, self.softcap, self.window, step.max_q_len,
                                                whole=whole, slopes=self.slopes)
            if a is None:
                a = ops.attn_prefill_paged(qkv, self.n_heads, self.n_kv, self.head_dim, line.k, line.v,
                                           line.page_table, line.page_size, line.ring, step.tok_pos, step.tok_slot,
                                           self.scale, self.softcap, self.window, slopes=self.slopes)
        elif step.mode == "prefill":
            a = ops.attn_prefill(qkv, self.n_heads, self.n_kv, self.head_dim, step.tok_pos, step.tok_row0,
                                 self.scale, self.softcap, self.window, step.seq_row0, step.seq_len, step.max_q_len,
                                 slopes=self.slopes)
        else:
            splits = self.decode_splits(step)
            n = step.n_seqs * self.n_heads * splits
            part = step.scratch.view(torch.float32)
            a = ops.attn_decode(qkv, self.n_heads, self.n_kv, self.head_dim, line.k, line.v, line.page_table,
                                line.page_size, line.ring, step.slots, line.slot_len, self.scale, self.softcap,
                                self.window, splits, part[:n * self.head_dim], part[n * self.head_dim:n * (self.head_dim + 2)],
                                slopes=self.slopes)
        return a
