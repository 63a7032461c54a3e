"""Each part alone against the plain implementation; the order list naming a layer twice and a
layer that reads another layer's cache; and toy parts defined here (a mixer with state of its
own, a feed-forward with routing, another position encoding) that are registered, built and
stepped without a change to the library's files."""
import json
import math
import os
from dataclasses import replace

import pytest
import torch

import plain_model
import replay
from tiny import TINY, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def _runtime(dtype, max_positions=256):
    from smolmoe_c99_b200.kernels import get_ops
    from smolmoe_c99_b200.parts import Runtime
    return Runtime(dtype=dtype, device=DEV, ops=get_ops(), max_positions=max_positions)


def _rand(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("size,eps", [(64, 1e-6), (96, 1e-5), (1000, 1e-3)])
def test_norm_part(dtype, size, eps):
    from smolmoe_c99_b200.config import PartSpec
    from smolmoe_c99_b200.parts import NORMS
    part = NORMS.get("rmsnorm")(PartSpec("rmsnorm", {"size": size, "eps": eps}, {"weight": "w"}), _runtime(dtype))
    assert [(s.name, s.shape, s.init) for s in part.param_specs(part.spec, "model.norm")] == [("model.norm.w", (size,), "ones")]
    w, x = (_rand((size,), 1, 0.3) + 1).to(dtype), _rand((7, size), 2, 3.0)
    part.bind({"weight": w.to(DEV)})
    want = plain_model.rmsnorm(x, w.float(), eps)
    got = part.forward(x.to(DEV)).float().cpu()
    assert float((got - want).abs().max()) <= (1e-5 if dtype == torch.float32 else 8e-3 * float(want.abs().max()))
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(part.forward(x.to(DEV), rows).float().cpu(), got[[5, 0, 5]])
    assert torch.equal(part.forward(x.to(DEV), lazy=True).tensor().float().cpu(), got)


@pytest.mark.parametrize("theta,rotary_dim", [(10000.0, 16), (1e6, 32), (50000.0, 48)])
def test_position_part(theta, rotary_dim):
    from smolmoe_c99_b200.config import PartSpec
    from smolmoe_c99_b200.parts import POSITIONS
    part = POSITIONS.get("rope")(PartSpec("rope", {"theta": theta, "rotary_dim": rotary_dim}), _runtime(torch.float32))
    cos, sin = part.tables(300)
    want_cos, want_sin = plain_model.rope_tables(300, rotary_dim, theta)
    assert torch.equal(cos.cpu(), want_cos) and torch.equal(sin.cpu(), want_sin)     # double angles, rounded once


def _gelu_tanh(g):
    return 0.5 * g * (1 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [5, 40, 300])
def test_feed_forward_part_with_another_activation(dtype, T):
    """tanh-GELU instead of SiLU: an entry of the activations the kernels know, through every kernel that folds the
    activation into the product (a handful of tokens, up to 64, more) and the stand-alone one of the 32-bit path."""
    from smolmoe_c99_b200.config import PartSpec
    from smolmoe_c99_b200.parts import FEED_FORWARDS
    D, H = 96, 160
    spec = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": H, "activation": "gelu_pytorch_tanh"},
                    {"gate": "mlp.g", "up": "mlp.u", "down": "mlp.d"})
    part = FEED_FORWARDS.get("gated_mlp")(spec, _runtime(dtype))
    g, u, d = (_rand(s, i, 0.1, dtype) for i, s in enumerate([(H, D), (H, D), (D, H)]))
    part.bind({"gate": g.to(DEV), "up": u.to(DEV), "down": d.to(DEV)})
    x, res = _rand((T, D), 5, 2.0, dtype), _rand((T, D), 6)
    want = res + (_gelu_tanh(x.float() @ g.float().T) * (x.float() @ u.float().T)) @ d.float().T
    got = res.to(DEV)
    part.forward(x.to(DEV), got, None)
    # bfloat16: the hidden activations are stored rounded (2^-9 of their size); against the largest output
    bound = 2e-5 if dtype == torch.float32 else 1e-2 * float(want.abs().max())
    assert float((got.cpu() - want).abs().max()) <= bound
    assert part.fused_decode_record() is None          # the whole-step kernel is written for SiLU


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from smolmoe_c99_b200.config import PartSpec
    from smolmoe_c99_b200.parts import FEED_FORWARDS
    D, H, T = 96, 160, 70
    spec = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": H, "activation": "silu"},
                    {"gate": "mlp.g", "up": "mlp.u", "down": "mlp.d"})
    part = FEED_FORWARDS.get("gated_mlp")(spec, _runtime(dtype))
    assert [(s.key, s.shape) for s in part.param_specs(spec, "l0")] == [("gate", (H, D)), ("up", (H, D)), ("down", (D, H))]
    g, u, d = (_rand(s, i, 0.1, dtype) for i, s in enumerate([(H, D), (H, D), (D, H)]))
    part.bind({"gate": g.to(DEV), "up": u.to(DEV), "down": d.to(DEV)})
    x, res = _rand((T, D), 5, 1.0, dtype), _rand((T, D), 6)
    want = res + plain_model.swiglu(x.float() @ g.float().T, x.float() @ u.float().T) @ d.float().T
    got = res.to(DEV)
    part.forward(x.to(DEV), got, None)
    assert float((got.cpu() - want).abs().max()) <= (2e-5 if dtype == torch.float32 else 2e-2)
    with pytest.raises(ValueError, match="activation"):
        FEED_FORWARDS.get("gated_mlp")(PartSpec("gated_mlp", dict(spec.params, activation="gelu"), spec.names), _runtime(dtype))


def _attention_reference(x, w, heads, kv_heads, hd, window, theta, lens):
    outs, at = [], 0
    for n in lens:
        xs = x[at:at + n]
        cos, sin = plain_model.rope_tables(n, hd, theta)
        q = plain_model.rope((xs @ w["q"].T + w["q_bias"]).view(n, heads, hd), cos, sin)
        k = plain_model.rope((xs @ w["k"].T + w["k_bias"]).view(n, kv_heads, hd), cos, sin)
        v = (xs @ w["v"].T + w["v_bias"]).view(n, kv_heads, hd)
        outs.append(plain_model.attend(q, k, v, heads, kv_heads, window).reshape(n, heads * hd) @ w["o"].T)
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,hd,window", [(4, 2, 16, None), (3, 1, 32, 20), (6, 3, 48, 70)])
def test_attention_part_prefill_then_decode(dtype, heads, kv_heads, hd, window):
    from smolmoe_c99_b200.cache import SequenceCache
    from smolmoe_c99_b200.config import PartSpec
    from smolmoe_c99_b200.engine.batch import pack_step
    from smolmoe_c99_b200.parts import MIXERS
    D, theta = 80, 20000.0
    spec = PartSpec("attention", {"hidden_size": D, "heads": heads, "kv_heads": kv_heads, "head_dim": hd, "qkv_bias": True,
                                  "window": window, "scale": 1 / math.sqrt(hd),
                                  "position": PartSpec("rope", {"theta": theta, "rotary_dim": hd})},
                    {k: k for k in ("q", "k", "v", "o", "q_bias", "k_bias", "v_bias")})
    cls = MIXERS.get("attention")
    part = cls(spec, _runtime(dtype))
    w = {s.key: _rand(s.shape, 10 + i, 0.15, dtype) for i, s in enumerate(cls.param_specs(spec, ""))}
    part.bind({k: t.to(DEV) for k, t in w.items()})
    wf = {k: t.float() for k, t in w.items()}
    need = cls.cache_need(spec)
    assert (need.kv_heads, need.head_dim, need.window) == (kv_heads, hd, window)
    cache = SequenceCache([need], max_tokens=1024, max_slots=4, max_seq_len=256, dtype=dtype, device=DEV)
    lens, extra = [1, 37, 90], 12
    total = [n + extra for n in lens]
    x_all = [_rand((n, D), 30 + i, 1.0, dtype) for i, n in enumerate(total)]
    want = [_attention_reference(x.float(), wf, heads, kv_heads, hd, window, theta, [len(x)]) for x in x_all]
    slots = [cache.alloc_slot() for _ in lens]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    # the prompts in one step
    step = pack_step(slots, [0] * 3, [[0] * n for n in lens], DEV)
    cache.reserve(dict(zip(slots, lens))); cache.flush_tables()
    res = torch.zeros((sum(lens), D), device=DEV)
    part.forward(torch.cat([x[:n] for x, n in zip(x_all, lens)]).to(DEV), res, step, cache.run_view(0))
    cache.advance(dict(zip(slots, lens)))
    got, at = res.cpu(), 0
    for i, n in enumerate(lens):
        assert float((got[at:at + n] - want[i][:n]).abs().max()) <= tol, f"prefill, sequence {i}"
        at += n
    # then one token each
    for j in range(extra):
        starts = [n + j for n in lens]
        step = pack_step(slots, starts, [[0]] * 3, DEV)
        cache.reserve({s: 1 for s in slots}); cache.flush_tables()
        res = torch.zeros((3, D), device=DEV)
        part.forward(torch.stack([x[s] for x, s in zip(x_all, starts)]).to(DEV), res, step, cache.run_view(0))
        cache.advance({s: 1 for s in slots})
        for i, s in enumerate(starts):
            assert float((res[i].cpu() - want[i][s]).abs().max()) <= tol, f"decode step {j}, sequence {i}"


# ---- the order list and cache sharing -----------------------------------------------------------
class SharedOrderConfig:
    """Model A's layers run in the order 0, 1, 1, 2 where layer 2 has no k/v projections and
    reads the cache of layer 0."""

    def __init__(self, base):
        self.base = base

    @classmethod
    def from_json(cls, raw):
        from smolmoe_c99_b200.config import Qwen2Config
        return cls(Qwen2Config.from_json(dict(raw, num_hidden_layers=3)))

    def to_json(self):
        return dict(self.base.to_json(), architectures=["SharedOrderForCausalLM"])

    def model_spec(self):
        from smolmoe_c99_b200.config import PartSpec
        spec = self.base.model_spec()
        last = spec.layers[2]
        mixer = PartSpec("attention", dict(last.mixer.params, kv_from_cache=True),
                         {k: v for k, v in last.mixer.names.items() if k[0] in "qo"})
        return replace(spec, architecture="SharedOrderForCausalLM", layers=(spec.layers[0], spec.layers[1],
                       replace(last, mixer=mixer, cache_from=0)), order=(0, 1, 1, 2))


def _plain_shared_order(model_dir, tokens):
    cfg = plain_model.read_config(model_dir)
    w = plain_model.read_safetensors(os.path.join(model_dir, "model.safetensors"))
    n, heads, kv_heads, hd = len(tokens), cfg["num_attention_heads"], cfg["num_key_value_heads"], plain_model.head_dim_of(cfg)
    cos, sin = plain_model.rope_tables(n, hd, cfg["rope_theta"])
    x = plain_model.embed(w["model.embed_tokens.weight"], tokens)
    kv0 = None
    for layer in (0, 1, 1, 2):
        p = f"model.layers.{layer}"
        y = plain_model.rmsnorm(x, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
        q = plain_model.rope((y @ w[f"{p}.self_attn.q_proj.weight"].T + w[f"{p}.self_attn.q_proj.bias"]).view(n, heads, hd), cos, sin)
        if layer == 2:
            k, v = kv0
        else:
            k = plain_model.rope((y @ w[f"{p}.self_attn.k_proj.weight"].T + w[f"{p}.self_attn.k_proj.bias"]).view(n, kv_heads, hd), cos, sin)
            v = (y @ w[f"{p}.self_attn.v_proj.weight"].T + w[f"{p}.self_attn.v_proj.bias"]).view(n, kv_heads, hd)
            if layer == 0:
                kv0 = (k, v)
        x = x + plain_model.attend(q, k, v, heads, kv_heads, None).reshape(n, heads * hd) @ w[f"{p}.self_attn.o_proj.weight"].T
        x = plain_model.ffn_block(x, w, p, cfg, None)
    return plain_model.rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T


def test_order_names_a_layer_twice_and_a_layer_reads_anothers_cache(tmp_path):
    from smolmoe_c99_b200.config import config_from_json, register_architecture
    from smolmoe_c99_b200.engine.engine import Engine
    from smolmoe_c99_b200.weights import write_random_model
    register_architecture("SharedOrderForCausalLM", SharedOrderConfig)
    cfg = config_from_json(dict(TINY["A"], architectures=["SharedOrderForCausalLM"]))
    folder = write_random_model(cfg, str(tmp_path / "m"), 3)
    names = set(json.loads(open(os.path.join(folder, "model.safetensors"), "rb").read()[8:8 + int.from_bytes(open(os.path.join(folder, "model.safetensors"), "rb").read(8), "little")]))
    assert "model.layers.2.self_attn.k_proj.weight" not in names and "model.layers.2.self_attn.q_proj.weight" in names
    engine = Engine(folder, "float32", max_tokens=1024)
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].n_layers == 3      # runs 0, 1 and 1 again own a cache
    requests = {f"r{i}": random_tokens(n, 256, 60 + i) for i, n in enumerate([3, 40, 77])}
    want = {r: _plain_shared_order(folder, t) for r, t in requests.items()}
    for cut, got in (("whole", replay.whole(engine, requests)), ("tail", replay.tail_decoded(engine, requests)),
                     ("batched", replay.batched(engine, [requests], {r: max(1, len(t) // 2) for r, t in requests.items()})),
                     ("portions", replay.portions(engine, requests, 7, 3))):
        for r in requests:
            assert float((got[r] - want[r]).abs().max()) <= 5e-6, f"{cut} {r}"


# ---- a toy mixer with state of its own -------------------------------------------------------------
def _register_toy():
    from smolmoe_c99_b200.parts import MIXERS, ParamSpec, Part, StateNeed, full_name

    @MIXERS.register("toy_decay")
    class ToyDecay(Part):
        """s_t = decay * s_(t-1) + x_t per sequence; adds s_t W^T to the residual."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.size, self.decay, self.w = int(spec["hidden_size"]), float(spec["decay"]), None

        @classmethod
        def param_specs(cls, spec, prefix):
            return [ParamSpec("w", full_name(prefix, spec.names["w"]), (int(spec["hidden_size"]),) * 2)]

        def bind(self, tensors):
            self.w = tensors["w"].float()

        @classmethod
        def cache_need(cls, spec):
            return StateNeed((int(spec["hidden_size"]),), torch.float32)

        def forward(self, x, residual, step, cache):
            assert cache.kind == "state"
            x = x.float()
            if step.mode == "decode":                      # one token per sequence: works inside a captured graph
                idx = step.slot_ids.long()
                s = cache.state.index_select(0, idx) * self.decay + x
                cache.state.index_copy_(0, idx, s)
                out = s
            else:
                out, at = torch.empty_like(x), 0
                for slot, n in zip(step.slots, step.seq_lens):
                    s = cache.state[slot]
                    for t in range(at, at + n):
                        s = s * self.decay + x[t]
                        out[t] = s
                    cache.state[slot] = s
                    at += n
            residual += out @ self.w.T
    return ToyDecay


class ToyConfig:
    def __init__(self, base):
        self.base = base

    @classmethod
    def from_json(cls, raw):
        from smolmoe_c99_b200.config import Qwen2Config
        return cls(Qwen2Config.from_json(raw))

    def to_json(self):
        return dict(self.base.to_json(), architectures=["ToyDecayForCausalLM"])

    def model_spec(self):
        from smolmoe_c99_b200.config import PartSpec
        spec = self.base.model_spec()
        toy = PartSpec("toy_decay", {"hidden_size": self.base.hidden_size, "decay": 0.75}, {"w": "toy_mixer.w"})
        return replace(spec, architecture="ToyDecayForCausalLM", layers=(spec.layers[0], replace(spec.layers[1], mixer=toy)))


def _plain_toy(model_dir, tokens):
    cfg = plain_model.read_config(model_dir)
    w = plain_model.read_safetensors(os.path.join(model_dir, "model.safetensors"))
    n = len(tokens)
    cos, sin = plain_model.rope_tables(n, plain_model.head_dim_of(cfg), cfg["rope_theta"])
    x = plain_model.embed(w["model.embed_tokens.weight"], tokens)
    x = plain_model.ffn_block(plain_model.attention_block(x, w, "model.layers.0", cfg, 0, cos, sin), w, "model.layers.0", cfg, None)
    y = plain_model.rmsnorm(x, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
    s, out = torch.zeros(cfg["hidden_size"]), torch.empty_like(y)
    for t in range(n):
        s = s * 0.75 + y[t]
        out[t] = s
    x = plain_model.ffn_block(x + out @ w["model.layers.1.toy_mixer.w"].T, w, "model.layers.1", cfg, None)
    return plain_model.rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from smolmoe_c99_b200.config import config_from_json, register_architecture
    from smolmoe_c99_b200.engine.engine import Engine
    from smolmoe_c99_b200.weights import write_random_model
    _register_toy()
    register_architecture("ToyDecayForCausalLM", ToyConfig)
    cfg = config_from_json(dict(TINY["A"], architectures=["ToyDecayForCausalLM"]))
    folder = write_random_model(cfg, str(tmp_path / "toy"), 9)
    engine = Engine(folder, "float32", max_tokens=1024, max_slots=3)
    assert len(engine.cache.states) == 1 and tuple(engine.cache.states[0].shape) == (3, 64)
    requests = {f"r{i}": random_tokens(n, 256, 20 + i) for i, n in enumerate([2, 35, 50, 64])}
    want = {r: _plain_toy(folder, t) for r, t in requests.items()}
    ids = list(requests)
    cuts = {"whole": replay.whole(engine, requests), "tail": replay.tail_decoded(engine, requests),
            "batched": replay.batched(engine, [{r: requests[r] for r in ids[:3]}, {r: requests[r] for r in ids[2:]}],
                                      {r: max(1, len(t) // 3) for r, t in requests.items()}),
            # a prompt in portions: the state goes on from where the portion before left it
            "portions": replay.portions(engine, requests, 9, 4),
            "joined": replay.joined(engine, {r: requests[r] for r in ids[:2]}, {r: requests[r] for r in ids[2:3]},
                                    {r: max(1, len(t) // 2) for r, t in requests.items()}, after=2, portion=5)}
    for cut, got in cuts.items():          # the state is carried from step to step and starts at zero in a used slot
        for r in got:
            assert float((got[r] - want[r]).abs().max()) <= 2e-5, f"{cut} {r}"


# ---- a toy feed-forward with routing, and another position encoding --------------------------------
def _register_toy_routed():
    from smolmoe_c99_b200.parts import FEED_FORWARDS, ParamSpec, Part, full_name

    @FEED_FORWARDS.register("toy_routed")
    class ToyRouted(Part):
        """Router logits in float over E square experts; each token goes to its best expert, whose
        output is weighted by that expert's softmax probability."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.size, self.experts = int(spec["hidden_size"]), int(spec["experts"])
            self.router = self.w = None

        @classmethod
        def param_specs(cls, spec, prefix):
            d, e = int(spec["hidden_size"]), int(spec["experts"])
            return [ParamSpec("router", full_name(prefix, spec.names["router"]), (e, d)),
                    ParamSpec("w", full_name(prefix, spec.names["experts"]), (e * d, d))]

        def bind(self, tensors):
            self.router, self.w = tensors["router"].float(), tensors["w"]

        def forward(self, x, residual, step):
            ops = self.runtime.ops
            logits = x.float() @ self.router.T                           # router logits in 32-bit
            prob, best = torch.softmax(logits, dim=-1).max(dim=-1)
            every = ops.linear(x, self.w, None, out_dtype=torch.float32)   # all experts through the library's product
            every = every.view(x.shape[0], self.experts, self.size)
            picked = every[torch.arange(x.shape[0], device=x.device), best]
            residual += picked * prob[:, None]
    return ToyRouted


def _register_toy_position():
    from smolmoe_c99_b200.parts import POSITIONS, Part

    @POSITIONS.register("toy_scaled_rope")
    class ScaledRotary(Part):
        """Rotary tables whose positions are divided by a factor (position interpolation)."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.theta, self.rotary_dim, self.factor = float(spec["theta"]), int(spec["rotary_dim"]), float(spec["factor"])
            self._tables = None

        def tables(self, n_positions):
            if self._tables is None or self._tables[0].shape[0] < n_positions:
                half = self.rotary_dim // 2
                inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                -(2.0 * torch.arange(half, dtype=torch.float64)) / self.rotary_dim)
                angle = (torch.arange(n_positions, dtype=torch.float64) / self.factor)[:, None] * inv[None, :]
                self._tables = (torch.cos(angle).float().to(self.runtime.device).contiguous(),
                                torch.sin(angle).float().to(self.runtime.device).contiguous())
            return self._tables
    return ScaledRotary


class ToyRoutedConfig:
    """Layer 0: attention under the scaled position encoding; layer 1: the routed feed-forward."""
    EXPERTS, FACTOR = 3, 4.0

    def __init__(self, base):
        self.base = base

    @classmethod
    def from_json(cls, raw):
        from smolmoe_c99_b200.config import Qwen2Config
        return cls(Qwen2Config.from_json(raw))

    def to_json(self):
        return dict(self.base.to_json(), architectures=["ToyRoutedForCausalLM"])

    def model_spec(self):
        from smolmoe_c99_b200.config import PartSpec
        spec = self.base.model_spec()
        l0, l1 = spec.layers
        old = l0.mixer.params["position"]
        scaled = PartSpec("toy_scaled_rope", dict(old.params, factor=self.FACTOR), old.names)
        mixer0 = replace(l0.mixer, params=dict(l0.mixer.params, position=scaled))
        routed = PartSpec("toy_routed", {"hidden_size": self.base.hidden_size, "experts": self.EXPERTS},
                          {"router": "toy_ffn.router", "experts": "toy_ffn.experts"})
        return replace(spec, architecture="ToyRoutedForCausalLM",
                       layers=(replace(l0, mixer=mixer0), replace(l1, feed_forward=routed)))


def _plain_toy_routed(model_dir, tokens):
    cfg = plain_model.read_config(model_dir)
    w = plain_model.read_safetensors(os.path.join(model_dir, "model.safetensors"))
    n, d, e = len(tokens), cfg["hidden_size"], ToyRoutedConfig.EXPERTS
    hd = plain_model.head_dim_of(cfg)
    half = hd // 2
    inv = torch.pow(torch.tensor(cfg["rope_theta"], dtype=torch.float64), -(2.0 * torch.arange(half, dtype=torch.float64)) / hd)
    angle = (torch.arange(n, dtype=torch.float64) / ToyRoutedConfig.FACTOR)[:, None] * inv[None, :]
    cos0, sin0 = torch.cos(angle).float(), torch.sin(angle).float()
    cos1, sin1 = plain_model.rope_tables(n, hd, cfg["rope_theta"])
    x = plain_model.embed(w["model.embed_tokens.weight"], tokens)
    x = plain_model.ffn_block(plain_model.attention_block(x, w, "model.layers.0", cfg, 0, cos0, sin0), w, "model.layers.0", cfg, None)
    x = plain_model.attention_block(x, w, "model.layers.1", cfg, 1, cos1, sin1)
    y = plain_model.rmsnorm(x, w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    prob, best = torch.softmax(y @ w["model.layers.1.toy_ffn.router"].T, dim=-1).max(dim=-1)
    experts = w["model.layers.1.toy_ffn.experts"].view(e, d, d)
    for t in range(n):
        x[t] = x[t] + prob[t] * (experts[best[t]] @ y[t])
    return plain_model.rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T


def test_a_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """Both are defined and registered here; the framework's files do not know them."""
    from smolmoe_c99_b200.config import config_from_json, register_architecture
    from smolmoe_c99_b200.engine.engine import Engine
    from smolmoe_c99_b200.weights import write_random_model
    _register_toy_routed()
    _register_toy_position()
    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
    cfg = config_from_json(dict(TINY["A"], architectures=["ToyRoutedForCausalLM"]))
    folder = write_random_model(cfg, str(tmp_path / "routed"), 11)
    engine = Engine(folder, "float32", max_tokens=1024, max_slots=3)
    requests = {f"r{i}": random_tokens(n, 256, 40 + i) for i, n in enumerate([3, 35, 50, 70])}
    want = {r: _plain_toy_routed(folder, t) for r, t in requests.items()}
    ids = list(requests)
    cuts = {"whole": replay.whole(engine, requests), "tail": replay.tail_decoded(engine, requests),
            "batched": replay.batched(engine, [{r: requests[r] for r in ids[:3]}, {r: requests[r] for r in ids[2:]}],
                                      {r: max(1, len(t) // 3) for r, t in requests.items()})}
    for cut, got in cuts.items():
        for r in got:
            assert float((got[r] - want[r]).abs().max()) <= 2e-5, f"{cut} {r}"


# ---- steps of a model that belong to no layer ----------------------------------------------------------------------
class ToyEndsConfig:
    """Model A with what a Qwen2 decoder does not have at its two ends: embeddings scaled by 8, a learned table of
    position vectors added to them, a bias on the output head, logits capped at 5, and tanh-GELU in layer 1's MLP."""
    SCALE, CAP = 8.0, 5.0

    def __init__(self, base):
        self.base = base

    @classmethod
    def from_json(cls, raw):
        from smolmoe_c99_b200.config import Qwen2Config
        return cls(Qwen2Config.from_json(raw))

    def to_json(self):
        return dict(self.base.to_json(), architectures=["ToyEndsForCausalLM"])

    def model_spec(self):
        from smolmoe_c99_b200.config import PartSpec
        spec = self.base.model_spec()
        l0, l1 = spec.layers
        gelu = replace(l1.feed_forward, params=dict(l1.feed_forward.params, activation="gelu_tanh"))
        table = PartSpec("learned", {"size": self.base.hidden_size, "positions": self.base.max_position_embeddings},
                         {"table": "weight"})
        return replace(spec, architecture="ToyEndsForCausalLM", layers=(l0, replace(l1, feed_forward=gelu)),
                       embedding_scale=self.SCALE, embedding_position=table, embedding_position_prefix="model.embed_positions",
                       head_bias_name="lm_head.bias", logit_softcap=self.CAP)


def _plain_toy_ends(model_dir, tokens):
    cfg = plain_model.read_config(model_dir)
    w = plain_model.read_safetensors(os.path.join(model_dir, "model.safetensors"))
    n = len(tokens)
    cos, sin = plain_model.rope_tables(n, plain_model.head_dim_of(cfg), cfg["rope_theta"])
    x = plain_model.embed(w["model.embed_tokens.weight"], tokens) * ToyEndsConfig.SCALE + w["model.embed_positions.weight"][:n]
    x = plain_model.ffn_block(plain_model.attention_block(x, w, "model.layers.0", cfg, 0, cos, sin), w, "model.layers.0", cfg, None)
    x = plain_model.attention_block(x, w, "model.layers.1", cfg, 1, cos, sin)
    y = plain_model.rmsnorm(x, w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    p = "model.layers.1.mlp"
    x = x + (_gelu_tanh(y @ w[f"{p}.gate_proj.weight"].T) * (y @ w[f"{p}.up_proj.weight"].T)) @ w[f"{p}.down_proj.weight"].T
    logits = plain_model.rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T + w["lm_head.bias"]
    return ToyEndsConfig.CAP * torch.tanh(logits / ToyEndsConfig.CAP)


def test_a_model_with_other_ends(tmp_path):
    """An embedding scale, added position vectors, a head bias and a cap on the logits are fields of the model's
    description, and another activation an entry of a table: an architecture defined here uses all of them."""
    from smolmoe_c99_b200.config import config_from_json, register_architecture
    from smolmoe_c99_b200.engine.engine import Engine
    from smolmoe_c99_b200.weights import write_random_model
    register_architecture("ToyEndsForCausalLM", ToyEndsConfig)
    cfg = config_from_json(dict(TINY["A"], architectures=["ToyEndsForCausalLM"]))
    folder = write_random_model(cfg, str(tmp_path / "ends"), 13)
    requests = {f"r{i}": random_tokens(n, 256, 80 + i) for i, n in enumerate([3, 40, 77])}
    want = {r: _plain_toy_ends(folder, t) for r, t in requests.items()}
    assert max(float(v.abs().max()) for v in want.values()) > 0.5            # the head bias and the scale make real logits
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 5e-2)):
        engine = Engine(folder, dtype, max_tokens=1024, max_slots=3)
        assert engine.model._fused_plan(engine.cache) is None                 # not the whole-step kernel's case
        for cut, got in (("whole", replay.whole(engine, requests)), ("tail", replay.tail_decoded(engine, requests)),
                         ("batched", replay.batched(engine, [requests], {r: max(1, len(t) // 2) for r, t in requests.items()})),
                         ("portions", replay.portions(engine, requests, 9, 4))):
            for r in requests:
                assert float((got[r] - want[r]).abs().max()) <= tol, f"{dtype} {cut} {r}"
