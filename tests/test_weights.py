"""Weights: the container, binding by name with one error for everything wrong, random weights (no GPU)."""
import json
import os
import struct

import pytest
import torch

from smolmoe_c99_b200.config import config_from_json
from smolmoe_c99_b200.engine.model import model_param_specs
from smolmoe_c99_b200.weights import (SafetensorsError, WeightsError, load_weights, open_checkpoint, write_random_model,
                                      write_safetensors)
from tiny import TINY

CPU = torch.device("cpu")


def _specs(name):
    return model_param_specs(config_from_json(TINY[name]).model_spec())


def _read_all(folder):
    return {n: st.tensor(n).clone() for n, (st, _) in open_checkpoint(folder).items()}


def test_random_weights_are_reproducible_and_as_specified(tmp_path):
    cfg = config_from_json(TINY["A"])
    a, b, c = (write_random_model(cfg, str(tmp_path / d), s) for d, s in (("a", 5), ("b", 5), ("c", 6)))
    ta, tb, tc = _read_all(a), _read_all(b), _read_all(c)
    assert all(torch.equal(ta[n], tb[n]) for n in ta)
    assert any(not torch.equal(ta[n], tc[n]) for n in ta)
    assert json.load(open(os.path.join(a, "config.json"))) == cfg.to_json()
    for n, t in ta.items():
        assert t.dtype == torch.bfloat16
        if "norm" in n:
            assert bool((t == 1).all())
        else:
            assert 0.015 < float(t.float().std()) < 0.025 and abs(float(t.float().mean())) < 0.005, n
    assert "lm_head.weight" not in ta                       # tied
    tb_cfg = config_from_json(TINY["B"])
    assert "lm_head.weight" in _read_all(write_random_model(tb_cfg, str(tmp_path / "B"), 1))   # untied


def test_dtypes_kept(model_dirs, tmp_path):
    specs = _specs("A")
    bf = load_weights(model_dirs["A"], specs, torch.bfloat16, CPU)
    assert all(t.dtype == torch.bfloat16 for t in bf.values())
    f32 = load_weights(model_dirs["A"], specs, torch.float32, CPU)
    assert all(t.dtype == torch.float32 for t in f32.values())
    assert all(torch.equal(f32[n], bf[n].float()) for n in bf)          # widening is exact
    # a tensor stored in 32-bit stays 32-bit in the bfloat16 engine; float16 becomes bfloat16
    tensors = _read_all(model_dirs["A"])
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() * 1.0001
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].to(torch.float16)
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    mixed = load_weights(str(tmp_path / "m"), specs, torch.bfloat16, CPU)
    assert mixed["model.norm.weight"].dtype == torch.float32
    assert mixed["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(model_dirs, tmp_path):
    tensors = _read_all(model_dirs["A"])
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)        # tied model: not expected
    tensors["model.layers.0.extra"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 127, dtype=torch.bfloat16)
    tensors["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"].to(torch.int32)
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_weights(str(tmp_path / "m"), _specs("A"), torch.bfloat16, CPU)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.self_attn.k_proj.bias", "model.norm.weight"]
    assert err.unexpected == ["lm_head.weight", "model.layers.0.extra"]
    assert len(err.wrong) == 2 and "expected [64, 128], found [64, 127]" in str(err) and "floating point" in str(err)
    for word in ("missing tensors (2)", "unexpected tensors (2)", "wrong shape or type (2)"):
        assert word in str(err)


def test_non_finite_weight_is_refused(model_dirs, tmp_path):
    tensors = _read_all(model_dirs["A"])
    tensors["model.layers.0.self_attn.q_proj.weight"][3, 3] = float("nan")
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    with pytest.raises(WeightsError, match="non-finite"):
        load_weights(str(tmp_path / "m"), _specs("A"), torch.bfloat16, CPU)


def test_malformed_containers(tmp_path):
    folder = tmp_path / "m"; os.makedirs(folder)
    path = folder / "model.safetensors"
    with pytest.raises(WeightsError, match="neither model.safetensors"):
        load_weights(str(folder), [], torch.bfloat16, CPU)
    path.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="truncated"):
        open_checkpoint(str(folder))
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        open_checkpoint(str(folder))
    path.write_bytes(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(SafetensorsError, match="not JSON"):
        open_checkpoint(str(folder))

    def with_header(h, payload=b"\0" * 16):
        blob = json.dumps(h).encode()
        path.write_bytes(struct.pack("<Q", len(blob)) + blob + payload)
    with_header({"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}})
    with pytest.raises(SafetensorsError, match="byte extent"):
        open_checkpoint(str(folder))
    with_header({"a": {"dtype": "BF16", "shape": [16], "data_offsets": [0, 32]}})
    with pytest.raises(SafetensorsError, match="past the end"):
        open_checkpoint(str(folder))
    with_header({"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 8]}, "b": {"dtype": "BF16", "shape": [4], "data_offsets": [4, 12]}})
    with pytest.raises(SafetensorsError, match="overlap"):
        open_checkpoint(str(folder))
    with_header({"a": {"dtype": "Q8", "shape": [4], "data_offsets": [0, 4]}})
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        open_checkpoint(str(folder))


def test_sharded_checkpoint(model_dirs, tmp_path):
    tensors = _read_all(model_dirs["A"])
    names = sorted(tensors)
    folder = tmp_path / "m"; os.makedirs(folder)
    halves = {"model-1.safetensors": names[: len(names) // 2], "model-2.safetensors": names[len(names) // 2:]}
    for fname, group in halves.items():
        write_safetensors(str(folder / fname), {n: tensors[n] for n in group})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {n: f for f, g in halves.items() for n in g}}))
    loaded = load_weights(str(folder), _specs("A"), torch.bfloat16, CPU)
    assert all(torch.equal(loaded[n], tensors[n]) for n in names)
