"""The attention mixer: q/k/v projections with bias, rotation of q and k, cache write,
causal attention over all keys or a window of them with grouped heads, output projection
added to the residual (reference: src/model.c:493-542; head-to-group map and window start:
src/model.c:459-472; scores, softmax and value sum: src/kernels.c:1138-1176).

Sizes and constants (hidden size, heads, groups, head size, window, scale, bias, position
encoding) are parameters of the part. With ``kv_from_cache`` the part has no k/v
projections of its own and attends over the cache of the run it is pointed at.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from .base import MIXERS, POSITIONS, KVNeed, ParamSpec, Part, Runtime, full_name


@MIXERS.register("attention")
class Attention(Part):
    takes_lazy_norm = True

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = spec.get("window")
        self.scale = float(spec["scale"])
        self.bias = bool(spec.get("qkv_bias", False))
        self.kv_from_cache = bool(spec.get("kv_from_cache", False))
        if self.heads % self.kv_heads:
            raise ValueError(f"kv_heads {self.kv_heads} must divide heads {self.heads}")
        if self.head_dim % 8 or self.head_dim > 256:
            # multiples of 16 up to 128 have tensor-core kernels; the other multiples of 8 run on the plain ones
            raise ValueError(f"head_dim {self.head_dim}: the attention kernels take multiples of 8 up to 256")
        pos_spec: PartSpec = spec["position"]
        self.position = POSITIONS.get(pos_spec.kind)(pos_spec, runtime)
        self.w_qkv = self.b_qkv = self.w_o = None

    # ---- weights -----------------------------------------------------------------------
    @classmethod
    def param_specs(cls, spec: PartSpec, prefix: str) -> List[ParamSpec]:
        d, hd = int(spec["hidden_size"]), int(spec["head_dim"])
        qd, kd = int(spec["heads"]) * hd, int(spec["kv_heads"]) * hd
        names = spec.names
        keys = [("q", qd)] if spec.get("kv_from_cache") else [("q", qd), ("k", kd), ("v", kd)]
        out = [ParamSpec(k, full_name(prefix, names[k]), (rows, d)) for k, rows in keys]
        out.append(ParamSpec("o", full_name(prefix, names["o"]), (d, qd)))
        if spec.get("qkv_bias"):
            out += [ParamSpec(k + "_bias", full_name(prefix, names[k + "_bias"]), (rows,)) for k, rows in keys]
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        keys = ["q"] if self.kv_from_cache else ["q", "k", "v"]
        # one product for q, k and v, as the reference computes them (src/model.c:506-509)
        self.w_qkv = torch.cat([tensors[k] for k in keys], dim=0).contiguous()
        self.b_qkv = torch.cat([tensors[k + "_bias"] for k in keys], dim=0).contiguous() if self.bias else None
        self.w_o = tensors["o"]

    @classmethod
    def cache_need(cls, spec: PartSpec):
        if spec.get("kv_from_cache"):
            return None
        return KVNeed(int(spec["kv_heads"]), int(spec["head_dim"]), spec.get("window"))

    # ---- one step ----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, step, cache) -> None:
        """``step.mode`` picks the kernels, not the function computed: ``prefill`` (every sequence at its first
        token) attends over the step's own packed keys, ``decode`` (one token each) over the cache, ``extend``
        (anything else) over the cache for earlier positions and the step's own keys for the rest."""
        ops, rt = self.runtime.ops, self.runtime
        T = x.shape[0]
        cos, sin = self.position.tables(rt.max_positions)
        own = not self.kv_from_cache
        mode = step.mode
        if cache.kind != "kv":
            raise RuntimeError("attention needs a key/value cache")
        if mode == "decode" and own:
            # one token per sequence: product, bias, rotation and cache write in one launch
            q = ops.qkv_rope_store_fused(x, self.w_qkv, self.b_qkv, step.positions, cos, sin, self.heads, self.kv_heads,
                                         self.head_dim, self.position.rotary_dim, cache.k_pool, cache.v_pool,
                                         cache.page_table, cache.ring, step.token_slot)
            if q is not None:
                ops.lap("qkv")   # with the norm before it, the rotation and the cache write
                att = ops.attention_cached(q, step, self.scale, self.window, cache, self.kv_heads)
                ops.lap("attention")
                ops.linear(att.view(T, self.heads * self.head_dim), self.w_o, None, out=residual, accumulate=True)
                ops.lap("attn_out")
                return
        # In a windowed group a new row takes the place of the row one ring earlier, which queries of this very step
        # may still see when sequences go on from the cache: those steps store after they have attended.
        store_late = own and mode == "extend" and cache.ring > 0
        write_now = own and not store_late
        where = dict(k_pool=cache.k_pool if write_now else None, v_pool=cache.v_pool if write_now else None,
                     page_table=cache.page_table, ring=cache.ring, token_slot=step.token_slot, token_end=step.token_end)
        # many tokens: product, bias, rotation and the cache write in one launch
        fused = ops.qkv_rope_store_many(x, self.w_qkv, self.b_qkv, step.positions, cos, sin, self.heads,
                                        self.kv_heads if own else 0, self.head_dim, self.position.rotary_dim,
                                        want_packed=own and mode != "decode", **where)
        if fused is not None:
            q, k_packed, v_packed = fused
            ops.lap("qkv")
        else:
            qkv = ops.linear(x, self.w_qkv, self.b_qkv, out_dtype=torch.float32)
            ops.lap("qkv")
            q, k_packed, v_packed = ops.rope_store(
                qkv, step.positions, cos, sin, self.heads, self.kv_heads if own else 0, self.head_dim,
                self.position.rotary_dim, rt.dtype, want_packed=own and mode != "decode", **where)
            ops.lap("rope")
        if own and mode == "prefill":
            att = ops.attention_prefill(q, k_packed, v_packed, step, self.scale, self.window)
        elif own and mode == "extend":
            att = ops.attention_extend(q, k_packed, v_packed, step, self.scale, self.window, cache, cache_written=write_now)
            if store_late:
                ops.kv_store(k_packed, v_packed, step, cache)
        else:
            if cache.ring and mode != "decode":
                self._check_ring_still_holds(step, cache)
            att = ops.attention_cached(q, step, self.scale, self.window, cache, self.kv_heads)
        ops.lap("attention")
        ops.linear(att.view(T, self.heads * self.head_dim), self.w_o, None, out=residual, accumulate=True)
        ops.lap("attn_out")

    def _check_ring_still_holds(self, step, cache) -> None:
        """A run that reads another run's windowed cache finds this step's rows already written: the oldest key a
        query of the step sees must not have been replaced by them."""
        starts = step.seq_starts if step.seq_starts is not None else [0] * step.n_seqs
        for start, n in zip(starts, step.seq_lens):
            oldest_needed = max(0, start - (self.window or cache.ring) + 1)
            if start + n - cache.ring > oldest_needed:
                raise RuntimeError(f"{n} tokens at position {start} have replaced keys of the windowed cache (ring "
                                   f"{cache.ring}) that the step's first query still sees: feed fewer tokens a step")

    def fused_decode_record(self, cache):
        """What a kernel that runs whole layers needs of this part and its cache, or None where the part is not the
        plain case that kernel is written for (keys and values of its own, every dimension rotated)."""
        if (type(self).forward is not Attention.forward or self.kv_from_cache or cache.kind != "kv"
                or self.position.rotary_dim != self.head_dim):
            return None
        cos, sin = self.position.tables(self.runtime.max_positions)
        return {"w_qkv": self.w_qkv, "b_qkv": self.b_qkv, "w_o": self.w_o, "hidden": self.hidden, "heads": self.heads,
                "kv_heads": self.kv_heads, "head_dim": self.head_dim, "scale": self.scale, "window": self.window or 0,
                "cos": cos, "sin": sin, "k_pool": cache.k_pool, "v_pool": cache.v_pool, "page_table": cache.page_table,
                "ring": cache.ring}
