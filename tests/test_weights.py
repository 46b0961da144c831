"""Weights: safetensors round trip, format errors, and the one error that lists
missing, unexpected and wrongly shaped tensors."""
import json
import os
import struct

import pytest
import torch

import helpers as H
from rust_inference_b200.engine.model import expected_tensors
from rust_inference_b200.config import config_from_dict
from rust_inference_b200.weights import (Checkpoint, SafetensorsError, WeightsError, load_checkpoint,
                                         save_safetensors, write_random_model)
from tiny_configs import TINY_A, TINY_B


def test_round_trip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4, 2).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.zeros(0, 4)}
    save_safetensors(str(tmp_path / "model.safetensors"), t)
    got = load_checkpoint(str(tmp_path), {n: tuple(x.shape) for n, x in t.items()})
    assert got["a"].dtype == torch.float32 and torch.equal(got["a"], t["a"])        # 32-bit stays 32-bit
    assert got["b"].dtype == torch.bfloat16 and torch.equal(got["b"], t["b"])       # bfloat16 stays bfloat16
    assert got["c"].dtype == torch.int32 and got["c"].tolist() == list(range(6))    # integer tables: int32
    assert got["d"].dtype == torch.float32 and torch.equal(got["d"], t["d"].float())
    assert got["e"].shape == (0, 4)


def test_one_error_lists_everything(tmp_path):
    d = H.make_model_dir(tmp_path, TINY_B, 1, stored="bfloat16")
    ck = Checkpoint(d)
    tensors = {n: ck.tensor(n).clone() for n in ck.names()}
    del tensors["model.layers.1.self_attn.q_norm.weight"]
    del tensors["model.layers.2.mlp.down_proj.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(96, 160)             # transposed
    tensors["model.norm.weight"] = torch.zeros(97)
    save_safetensors(os.path.join(d, "model.safetensors"), tensors)
    spec = config_from_dict(TINY_B).to_spec()
    with pytest.raises(WeightsError) as ei:
        load_checkpoint(d, {n: i.shape for n, i in expected_tensors(spec).items()})
    e = ei.value
    assert e.missing == ["model.layers.1.self_attn.q_norm.weight", "model.layers.2.mlp.down_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.mlp.gate_proj.weight", "model.norm.weight"]
    for needle in ("q_norm", "down_proj", "q_proj.bias", "[96, 160]", "[160, 96]", "[97]"):
        assert needle in str(e)


def test_tied_and_absent_head(tmp_path, emulated_ops):
    from rust_inference_b200.engine import Model
    # tied: no lm_head tensor is written, and one that is present anyway is ignored
    d = H.make_model_dir(tmp_path, TINY_A, 2, stored="float32", name="tied")
    assert "lm_head.weight" not in Checkpoint(d)
    m = Model.from_dir(d, "float32", "cpu")
    assert m.head is m.embedding
    # untied config whose checkpoint lacks the head: tied, as the reference does (qwen3.rs:166-171 there)
    d2 = H.make_model_dir(tmp_path, TINY_B, 2, stored="bfloat16", name="untied")
    ck = Checkpoint(d2)
    tensors = {n: ck.tensor(n).clone() for n in ck.names() if n != "lm_head.weight"}
    save_safetensors(os.path.join(d2, "model.safetensors"), tensors)
    m2 = Model.from_dir(d2, "float32", "cpu")
    assert m2.head is m2.embedding
    assert m2.embedding.dtype == torch.float32        # stored bfloat16, computing in float32


def test_format_errors(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too small"):
        Checkpoint(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header"):
        Checkpoint(str(tmp_path))
    h = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="offsets"):
        Checkpoint(str(tmp_path))
    h = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="dtype"):
        Checkpoint(str(tmp_path))
    os.remove(p)
    with pytest.raises(SafetensorsError, match="neither"):
        Checkpoint(str(tmp_path))


def test_sharded_index(tmp_path):
    save_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.ones(2)})
    save_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    got = load_checkpoint(str(tmp_path), {"a": (2,), "b": (3,)})
    assert got["a"].tolist() == [1, 1] and got["b"].tolist() == [0, 0, 0]


def test_random_mode_is_seeded_and_in_distribution(tmp_path):
    a = write_random_model(dict(TINY_B), 5, str(tmp_path / "a"), dtype="float32")
    b = write_random_model(dict(TINY_B), 5, str(tmp_path / "b"), dtype="float32")
    c = write_random_model(dict(TINY_B), 6, str(tmp_path / "c"), dtype="float32")
    A, B, C = Checkpoint(a), Checkpoint(b), Checkpoint(c)
    spec = config_from_dict(TINY_B).to_spec()
    assert sorted(A.names()) == sorted(expected_tensors(spec))
    for n in A.names():
        assert torch.equal(A.tensor(n), B.tensor(n))
    assert not torch.equal(A.tensor("lm_head.weight"), C.tensor("lm_head.weight"))
    w = A.tensor("model.embed_tokens.weight")
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    for n in ("model.norm.weight", "model.layers.0.self_attn.k_norm.weight"):
        g = A.tensor(n)
        assert float(g.min()) >= 0.9 and float(g.max()) <= 1.1 and float(g.std()) > 0.01
    with open(os.path.join(a, "config.json")) as f:
        assert json.load(f)["hidden_size"] == 96


def test_random_weights_are_a_function_of_seed_name_and_index():
    """The host code gives, bit for bit, what the rule written out in numpy gives; rows of a tensor can be made
    alone; another name or seed gives other values; the moments are those of N(0, 0.02) and 1 + U(-0.1, 0.1)."""
    import numpy as np
    import plain_random as pr
    from rust_inference_b200.weights.random_init import random_tensor, tensor_key
    assert tensor_key(7, "model.norm.weight") == pr.tensor_key(7, "model.norm.weight")
    w = random_tensor(7, "w", (400, 333), "matrix", torch.float32)
    assert np.array_equal(w.numpy(), pr.normal(pr.tensor_key(7, "w"), np.arange(400 * 333)).reshape(400, 333))
    assert torch.equal(random_tensor(7, "w", (5, 333), "matrix", torch.float32, first_row=123), w[123:128])
    assert torch.equal(random_tensor(7, "w", (400, 333), "matrix", torch.bfloat16), w.to(torch.bfloat16))
    g = random_tensor(7, "g", (50000,), "gain", torch.float32)
    assert np.array_equal(g.numpy(), pr.uniform(pr.tensor_key(7, "g"), np.arange(50000)))
    assert not torch.equal(random_tensor(7, "v", (400, 333), "matrix", torch.float32), w)
    assert not torch.equal(random_tensor(8, "w", (400, 333), "matrix", torch.float32), w)
    z = (w.double() / 0.02).flatten()
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1) < 0.01 and abs(float((z ** 4).mean()) - 3) < 0.1
    assert 0.9 <= float(g.min()) < 0.9001 and 1.0999 < float(g.max()) <= 1.1 and abs(float(g.mean()) - 1) < 1e-3
    assert random_tensor(7, "t", (3, 4), "table", torch.float32).dtype == torch.int32


@pytest.mark.gpu
def test_random_weights_host_and_device_agree():
    """The device kernel and the host code give the same bits, in float32 and in bfloat16, for whole tensors and
    for rows in the middle of one: a model made on the device is the model that the host would have written."""
    from rust_inference_b200.weights.random_init import random_tensor
    for dtype in (torch.float32, torch.bfloat16):
        for role, shape in (("matrix", (3000, 777)), ("gain", (4097,)), ("matrix", (1, 5))):
            host = random_tensor(11, "x", shape, role, dtype)
            dev = random_tensor(11, "x", shape, role, dtype, device="cuda")
            assert torch.equal(host, dev.cpu()), (dtype, role, shape)
        rows = random_tensor(11, "x", (40, 777), "matrix", dtype, device="cuda", first_row=2900)
        assert torch.equal(rows.cpu(), random_tensor(11, "x", (3000, 777), "matrix", dtype)[2900:2940])
