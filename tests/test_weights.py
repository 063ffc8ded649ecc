"""Safetensors reading, binding by name, errors, and the random-weights folder (CPU)."""
import json
import os

import pytest
import torch

from hi_b200.config import lookup
from hi_b200.parts.model import Model
from hi_b200.weights import (Checkpoint, SafetensorsError, WeightError, check_names, load_from_dir,
                             write_random_model, write_safetensors)
from tiny_configs import TINY_A, TINY_B


def fake_model(cfg, dtype=torch.bfloat16):
    arch = lookup(cfg)
    model = Model(arch.build_spec(arch.parse_config(cfg, None)), dtype, "cpu")
    return arch, model


def test_roundtrip_against_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32),
               "f": torch.randn(2, 2, 2), "h": torch.randn(4).to(torch.float16)}
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    theirs = load_file(str(tmp_path / "model.safetensors"))
    for k, v in tensors.items():
        assert torch.equal(theirs[k], v)
    os.makedirs(tmp_path / "x")
    save_file(tensors, str(tmp_path / "x" / "model.safetensors"))
    mine = Checkpoint(str(tmp_path / "x"))
    assert sorted(mine.names()) == sorted(tensors)
    for k, v in tensors.items():
        assert torch.equal(mine.tensor(k), v) and mine.describe(k) == ({torch.bfloat16: "BF16", torch.int32: "I32",
                                                                        torch.float32: "F32", torch.float16: "F16"}[v.dtype], tuple(v.shape))


def test_random_folder_is_seeded_and_complete(tmp_path):
    d1 = write_random_model(TINY_A, str(tmp_path / "a1"), seed=5)
    d2 = write_random_model(TINY_A, str(tmp_path / "a2"), seed=5)
    d3 = write_random_model(TINY_A, str(tmp_path / "a3"), seed=6)
    c1, c2, c3 = Checkpoint(d1), Checkpoint(d2), Checkpoint(d3)
    assert json.load(open(os.path.join(d1, "config.json"))) == TINY_A
    for n in c1.names():
        assert c1.describe(n)[0] == "BF16"
        assert torch.equal(c1.tensor(n), c2.tensor(n))
    assert not torch.equal(c1.tensor("model.layers.0.self_attn.q_proj.weight"), c3.tensor("model.layers.0.self_attn.q_proj.weight"))
    assert bool((c1.tensor("model.norm.weight") == 1).all())
    q = c1.tensor("model.layers.0.self_attn.q_proj.weight").float()
    assert abs(float(q.std()) - 0.02) < 0.003
    assert c1.describe("model.layers.1.feed_forward.experts.down_proj.weight")[1] == (4, 64, 128)
    assert "lm_head.weight" in c1.names()
    db = write_random_model(TINY_B, str(tmp_path / "b"), seed=1)
    assert "lm_head.weight" not in Checkpoint(db).names()          # tied head: no tensor written


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(TINY_A, str(tmp_path / "m"), seed=1)
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    del tensors["model.layers.1.self_attn.k_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.embed_tokens.weight"] = torch.zeros(255, 64, dtype=torch.bfloat16)
    tensors["vision_model.patch.weight"] = torch.zeros(2)           # not the text decoder: ignored
    tensors["language_model.model.layers.0.input_layernorm.weight"] = tensors.pop("model.layers.0.input_layernorm.weight")
    bad = str(tmp_path / "bad")
    os.makedirs(bad)
    write_safetensors(os.path.join(bad, "model.safetensors"), tensors)
    json.dump(TINY_A, open(os.path.join(bad, "config.json"), "w"))
    arch, model = fake_model(TINY_A)
    with pytest.raises(WeightError) as e:
        load_from_dir(model, bad, arch.normalize_tensor_name)
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.embed_tokens.weight"]
    text = str(err)
    for word in ("k_proj", "model.norm.weight", "extra.weight", "[255, 64]", "[256, 64]"):
        assert word in text


def test_dtypes_kept_as_stored(tmp_path):
    """BF16 stays bfloat16, F16 becomes bfloat16, a tensor stored in 32-bit stays 32-bit; the
    float32 path widens everything."""
    d = write_random_model(TINY_A, str(tmp_path / "m"), seed=1)
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() * 1.5
    tensors["model.layers.0.input_layernorm.weight"] = tensors["model.layers.0.input_layernorm.weight"].to(torch.float16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    arch, model = fake_model(TINY_A, torch.bfloat16)
    load_from_dir(model, d, arch.normalize_tensor_name)
    assert model.final_norm.weight.dtype == torch.float32 and float(model.final_norm.weight[0]) == 1.5
    assert model.layers[0].norm_mixer.weight.dtype == torch.bfloat16
    assert model.embedding.table.dtype == torch.bfloat16
    assert model.layers[0].mixer.w_qkv.shape == ((4 + 2 * 2) * 16, 64)
    arch, m32 = fake_model(TINY_A, torch.float32)
    load_from_dir(m32, d, arch.normalize_tensor_name)
    assert m32.embedding.table.dtype == torch.float32 and m32.layers[1].feed_forward.w_gate.dtype == torch.float32


def test_container_errors(tmp_path):
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        Checkpoint(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00\x00\x00\x00\x00\x00\x00{bad}")
    with pytest.raises(SafetensorsError, match="JSON"):
        Checkpoint(str(tmp_path))
    (tmp_path / "model.safetensors").write_bytes(b"\xff\xff\xff\xff\x00\x00\x00\x00{}")
    with pytest.raises(SafetensorsError, match="header length"):
        Checkpoint(str(tmp_path))
    # a quantized companion tensor is refused by name
    header = json.dumps({"w.scales": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(len(header).to_bytes(8, "little") + header + b"\0\0")
    with pytest.raises(SafetensorsError, match="quantized"):
        ck = Checkpoint(str(tmp_path)); ck.tensor("w.scales")


def test_sharded_checkpoint_with_index(tmp_path):
    d = write_random_model(TINY_A, str(tmp_path / "m"), seed=2)
    ck = Checkpoint(d)
    names = sorted(ck.names())
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    sharded = tmp_path / "sharded"
    os.makedirs(sharded)
    for fname, ns in parts.items():
        write_safetensors(str(sharded / fname), {n: ck.tensor(n).clone() for n in ns})
    json.dump({"weight_map": {n: f for f, ns in parts.items() for n in ns}}, open(sharded / "model.safetensors.index.json", "w"))
    json.dump(TINY_A, open(sharded / "config.json", "w"))
    arch, model = fake_model(TINY_A)
    load_from_dir(model, str(sharded), arch.normalize_tensor_name)
    assert torch.equal(model.embedding.table, ck.tensor("model.embed_tokens.weight"))


def test_random_values_are_the_written_out_definition_and_look_normal():
    """The host runtime's generator against the same arithmetic written out in numpy; values are
    a function of (seed, name, element index) alone; their moments are a normal distribution's."""
    import numpy as np

    from hi_b200.weights import random_values as rv

    key = rv.tensor_key(7, "model.layers.0.self_attn.q_proj.weight")
    a = rv.normal_values(key, 0, 70001, 0.02)
    b = rv.normal_values_numpy(key, 0, 70001, 0.02)
    assert a.dtype == np.float32 and (a.view(np.uint32) == b.view(np.uint32)).all()
    assert (rv.normal_values(key, 12345, 100, 0.02) == a[12345:12445]).all(), "a value depends on more than its index"
    assert rv.tensor_key(7, "x") != rv.tensor_key(8, "x") != rv.tensor_key(8, "y")
    other = rv.normal_values(rv.tensor_key(8, "model.layers.0.self_attn.q_proj.weight"), 0, 70001, 0.02)
    assert abs(float(np.corrcoef(a, other)[0, 1])) < 0.02
    big = rv.normal_values(key, 0, 2_000_000, 1.0).astype(np.float64)
    assert abs(big.mean()) < 3e-3 and abs(big.std() - 1.0) < 3e-3
    assert abs((big ** 3).mean()) < 1e-2 and abs((big ** 4).mean() - 3.0) < 3e-2
    assert 4.0 < np.abs(big).max() < 16.1
    # consecutive elements are not correlated
    assert abs(float(np.corrcoef(big[:-1], big[1:])[0, 1])) < 3e-3


def test_random_model_is_a_function_of_the_seed(tmp_path):
    d1 = write_random_model(TINY_A, str(tmp_path / "a"), seed=5, std=0.02)
    d2 = write_random_model(TINY_A, str(tmp_path / "b"), seed=5, std=0.02)
    d3 = write_random_model(TINY_A, str(tmp_path / "c"), seed=6, std=0.02)
    c1, c2, c3 = Checkpoint(d1), Checkpoint(d2), Checkpoint(d3)
    name = "model.layers.1.feed_forward.experts.up_proj.weight"
    assert torch.equal(c1.tensor(name), c2.tensor(name)) and not torch.equal(c1.tensor(name), c3.tensor(name))
    assert torch.equal(c1.tensor("model.norm.weight"), torch.ones(64, dtype=torch.bfloat16))
    assert abs(float(c1.tensor(name).float().std()) - 0.02) < 1e-3


def test_fused_expert_layout_and_biases_by_presence(tmp_path):
    """The routed experts stored as one fused, input-major tensor per layer without a ``.weight``
    suffix (``experts.gate_up_proj`` [E, H, 2I], ``experts.down_proj`` [E, I, H]) load into the same
    weights as the converted layout; q/k/v/o biases are used iff their tensors exist; a fused
    tensor of the wrong shape is reported by the name the model asks for."""
    d = write_random_model(TINY_A, str(tmp_path / "m"), seed=9)
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    fused = {}
    for n, t in tensors.items():
        if n.endswith("experts.gate_proj.weight"):
            up = tensors[n.replace("gate_proj", "up_proj")]
            fused[n.replace("gate_proj.weight", "gate_up_proj")] = torch.cat([t, up], dim=1).transpose(1, 2).contiguous()
        elif n.endswith("experts.up_proj.weight"):
            continue
        elif n.endswith("experts.down_proj.weight"):
            fused[n[: -len(".weight")]] = t.transpose(1, 2).contiguous()
        else:
            fused[n] = t
    fused["model.layers.0.self_attn.k_proj.bias"] = torch.full((2 * 16,), 0.5, dtype=torch.bfloat16)
    out = tmp_path / "fused"
    os.makedirs(out)
    write_safetensors(str(out / "model.safetensors"), fused)
    json.dump(TINY_A, open(out / "config.json", "w"))
    arch, plain_model = fake_model(TINY_A)
    load_from_dir(plain_model, d, arch.normalize_tensor_name, arch.derive_tensors)
    arch, model = fake_model(TINY_A)
    load_from_dir(model, str(out), arch.normalize_tensor_name, arch.derive_tensors)
    for a, b in zip(plain_model.layers, model.layers):
        for w in ("w_gate", "w_up", "w_down"):
            assert torch.equal(getattr(a.feed_forward, w), getattr(b.feed_forward, w)), w
    assert plain_model.layers[0].mixer.b_qkv is None and model.layers[1].mixer.b_qkv is None
    b_qkv = model.layers[0].mixer.b_qkv
    assert b_qkv.shape == ((4 + 2 + 2) * 16,) and float(b_qkv[: 4 * 16].abs().max()) == 0.0
    assert torch.equal(b_qkv[4 * 16: 6 * 16], torch.full((32,), 0.5, dtype=torch.bfloat16))
    # a fused tensor of the wrong width
    fused["model.layers.0.feed_forward.experts.down_proj"] = torch.zeros(4, 100, 64, dtype=torch.bfloat16)
    write_safetensors(str(out / "model.safetensors"), fused)
    arch, model = fake_model(TINY_A)
    with pytest.raises(WeightError) as e:
        load_from_dir(model, str(out), arch.normalize_tensor_name, arch.derive_tensors)
    assert e.value.wrong_shape and e.value.wrong_shape[0][0] == "model.layers.0.feed_forward.experts.down_proj.weight"
