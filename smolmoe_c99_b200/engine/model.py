"""The decoder put together from a ``ModelSpec``: embedding, the layers' blocks in the order
the spec lists them, final norm and output head (reference: src/model.c:664-690 for the
forward pass, src/model.c:654-662 for the head on the wanted rows only)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..parts import BLOCKS, NORMS, POSITIONS, ParamSpec, Runtime, full_name


def model_param_specs(spec: ModelSpec) -> List[ParamSpec]:
    """Every tensor the model needs, by name and shape."""
    out = [ParamSpec("embedding", spec.embedding_name, (spec.vocab_size, spec.hidden_size))]
    for layer in spec.layers:
        out += BLOCKS.get(layer.block).param_specs(layer)
    out += NORMS.get(spec.final_norm.kind).param_specs(spec.final_norm, spec.final_norm_prefix)
    if spec.head_name is not None:
        out.append(ParamSpec("head", spec.head_name, (spec.vocab_size, spec.hidden_size)))
    if spec.head_bias_name is not None:
        out.append(ParamSpec("head_bias", spec.head_bias_name, (spec.vocab_size,)))
    if spec.embedding_position is not None:
        out += POSITIONS.get(spec.embedding_position.kind).param_specs(spec.embedding_position, spec.embedding_position_prefix)
    names = [s.name for s in out]
    if len(set(names)) != len(names):
        dup = sorted({n for n in names if names.count(n) > 1})
        raise ValueError(f"the model names a tensor twice: {', '.join(dup)}")
    return out


def cache_needs(spec: ModelSpec) -> list:
    """What each run of ``spec.order`` needs from the cache (see ``SequenceCache``)."""
    needs: list = []
    last_run_of: Dict[int, int] = {}
    for run, index in enumerate(spec.order):
        layer = spec.layers[index]
        if layer.cache_from is not None:
            if layer.cache_from not in last_run_of:
                raise ValueError(f"layer {index} reads the cache of layer {layer.cache_from}, which has not run before it")
            needs.append(last_run_of[layer.cache_from])
        else:
            needs.append(BLOCKS.get(layer.block).cache_need(layer))
        last_run_of[index] = run
    return needs


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.blocks = [BLOCKS.get(layer.block)(layer, runtime) for layer in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, runtime)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.head_bias: Optional[torch.Tensor] = None
        self.embedding_position = None
        if spec.embedding_position is not None:
            self.embedding_position = POSITIONS.get(spec.embedding_position.kind)(spec.embedding_position, runtime)
            if not hasattr(self.embedding_position, "add_to"):
                raise ValueError(f"position encoding {spec.embedding_position.kind!r} cannot be added to the embeddings "
                                 f"(it has no add_to)")
        self._fused = {}     # per cache: what the fused decode step needs, or None where the model is not its case

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embedding = tensors[self.spec.embedding_name]
        for block in self.blocks:
            block.bind(tensors)
        norm_specs = type(self.final_norm).param_specs(self.spec.final_norm, self.spec.final_norm_prefix)
        self.final_norm.bind({s.key: tensors[s.name] for s in norm_specs})
        # a tied head is the same device buffer as the embedding (src/modelfile.c:25-34)
        self.head = self.embedding if self.spec.head_name is None else tensors[self.spec.head_name]
        self.head_bias = tensors[self.spec.head_bias_name] if self.spec.head_bias_name is not None else None
        if self.embedding_position is not None:
            pos_specs = type(self.embedding_position).param_specs(self.spec.embedding_position, self.spec.embedding_position_prefix)
            self.embedding_position.bind({s.key: tensors[s.name] for s in pos_specs})

    def _plain_ends(self) -> bool:
        """Whether the model's first and last steps are the plain ones: embedding, final norm, head."""
        s = self.spec
        return s.embedding_scale == 1.0 and s.embedding_position is None and s.head_bias_name is None and s.logit_softcap is None

    # ---- a decode step of standard layers in one kernel ---------------------------------------------------
    def _fused_plan(self, cache):
        """The layer records of the fused decode step for this cache, built once: every run of ``order`` must be a
        layer whose parts describe themselves to that kernel, all with the same sizes, in bfloat16."""
        key = id(cache)
        if key in self._fused:
            return self._fused[key]
        self._fused[key] = None
        ops, rt = self.runtime.ops, self.runtime
        if rt.dtype != torch.bfloat16 or not hasattr(self.final_norm, "fused_decode_record") or not self._plain_ends():
            return None
        records = []
        for run, index in enumerate(self.spec.order):
            block = self.blocks[index]
            rec = block.fused_decode_record(cache.run_view(run)) if hasattr(block, "fused_decode_record") else None
            if rec is None:
                return None
            records.append(rec)
        final = self.final_norm.fused_decode_record()
        if final is None or not records:
            return None
        m0, f0 = records[0]["mixer"], records[0]["ffn"]
        sizes = {"D": m0["hidden"], "H": f0["intermediate"], "heads": m0["heads"], "kv_heads": m0["kv_heads"],
                 "head_dim": m0["head_dim"], "V": self.spec.vocab_size}
        tensors = [self.embedding, self.head, final[0]]
        for rec in records:
            m, f = rec["mixer"], rec["ffn"]
            same = (m["hidden"], m["heads"], m["kv_heads"], m["head_dim"], m["scale"], f["hidden"], f["intermediate"]) == \
                   (sizes["D"], sizes["heads"], sizes["kv_heads"], sizes["head_dim"], m0["scale"], sizes["D"], sizes["H"])
            if not same or m["k_pool"].dtype != torch.bfloat16:
                return None
            tensors += [m["w_qkv"], m["w_o"], f["w_gate_up"], f["w_down"], rec["norm1"][0], rec["norm2"][0]]
            if m["b_qkv"] is not None:
                tensors.append(m["b_qkv"])
        if any(t.dtype != torch.bfloat16 or not t.is_contiguous() for t in tensors):
            return None
        if ops.decode_fused_refusal(1, sizes["D"], sizes["H"], sizes["heads"], sizes["kv_heads"], sizes["head_dim"], sizes["V"]):
            return None
        from ..kernels.ops import FusedLayerRecord
        import ctypes
        table = (FusedLayerRecord * len(records))()
        for out, rec in zip(table, records):
            m, f = rec["mixer"], rec["ffn"]
            out.w_qkv, out.w_o, out.w_gate_up, out.w_down = m["w_qkv"].data_ptr(), m["w_o"].data_ptr(), f["w_gate_up"].data_ptr(), f["w_down"].data_ptr()
            out.b_qkv = m["b_qkv"].data_ptr() if m["b_qkv"] is not None else None
            out.norm1, out.norm2 = rec["norm1"][0].data_ptr(), rec["norm2"][0].data_ptr()
            out.k_pool, out.v_pool, out.page_table = m["k_pool"].data_ptr(), m["v_pool"].data_ptr(), m["page_table"].data_ptr()
            out.cos_table, out.sin_table = m["cos"].data_ptr(), m["sin"].data_ptr()
            out.table_stride, out.ring, out.window = m["page_table"].shape[1], m["ring"], m["window"]
            out.eps1, out.eps2 = rec["norm1"][1], rec["norm2"][1]
        layers = torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8).to(rt.device)
        weights = [w for rec in records for w in (rec["mixer"]["w_qkv"], rec["mixer"]["w_o"], rec["ffn"]["w_gate_up"],
                                                   rec["ffn"]["w_down"])] + [self.head]
        maps, bk = ops.decode_fused_maps(weights, sizes, rt.device)
        plan = {"layers": layers, "maps": maps, "bk": bk, "n_layers": len(records), "sizes": sizes, "norm_f": final[0], "eps_f": final[1],
                "scale": m0["scale"], "keep": records,
                "scratch": ops.decode_fused_scratch(sizes["D"], sizes["H"], sizes["heads"], sizes["kv_heads"],
                                                    sizes["head_dim"], sizes["V"], rt.device)}
        self._fused[key] = plan
        return plan

    def forward(self, step, cache, want_rows: Optional[torch.Tensor], status: Optional[torch.Tensor] = None):
        """Runs the step's tokens through every layer; returns float logits ``[wanted, vocab]``
        for the packed token indices in ``want_rows`` (int32), or None when none are wanted."""
        ops = self.runtime.ops
        if (step.mode == "decode" and step.n_tokens <= 16 and getattr(ops, "use_fused_decode", False)
                and ops.phase_times is None):
            plan = self._fused_plan(cache)
            if plan is not None and not ops.decode_fused_refusal(step.n_tokens, *[plan["sizes"][k] for k in
                                                                 ("D", "H", "heads", "kv_heads", "head_dim", "V")]):
                rows = want_rows if want_rows is not None and want_rows.numel() else None
                return ops.decode_fused(plan["layers"], plan["maps"], plan["bk"], plan["n_layers"], plan["sizes"], self.embedding, self.head,
                                        plan["norm_f"], plan["eps_f"], plan["scale"], step.tokens, step.positions,
                                        step.token_slot, rows, plan["scratch"], status)
        ops.lap(None)
        residual = ops.embedding(self.embedding, step.tokens, status)
        if self.spec.embedding_scale != 1.0:
            ops.scale_(residual, self.spec.embedding_scale)
        if self.embedding_position is not None:
            self.embedding_position.add_to(residual, step)
        ops.lap("embed")
        for run, index in enumerate(self.spec.order):
            self.blocks[index].forward(residual, step, cache.run_view(run))
        if want_rows is None or want_rows.numel() == 0:
            return None
        every_row = getattr(step, "wants_every_row", False)   # the wanted rows are 0..T-1 in order
        x = self.final_norm.forward(residual, None if every_row else want_rows, lazy=True)
        logits = ops.linear(x, self.head, self.head_bias, out_dtype=torch.float32)
        if self.spec.logit_softcap is not None:
            ops.softcap_(logits, self.spec.logit_softcap)
        ops.lap("logits")
        return logits

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (a tied head counts once)."""
        seen, total = set(), 0
        tensors = [self.embedding if self.head is self.embedding else self.head, self.head_bias]
        if self.embedding_position is not None:
            tensors += [v for v in vars(self.embedding_position).values() if isinstance(v, torch.Tensor)]
        for block in self.blocks:
            for part in (block.mixer_norm, block.mixer, block.feed_forward_norm, block.feed_forward):
                tensors += [v for v in vars(part).values() if isinstance(v, torch.Tensor)]
        tensors += [v for v in vars(self.final_norm).values() if isinstance(v, torch.Tensor)]
        for t in tensors:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total
