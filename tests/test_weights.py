"""safetensors reading and writing, the by-name loader's one error, random weights."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_gpt2
from conftest import TINY_A, TINY_B
from math_utils_b200.config import Gpt2Config
from math_utils_b200.engine.assemble import collect_tensor_specs
from math_utils_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights,
                                     write_random_model, write_safetensors)


def test_round_trip_and_own_reader_agree(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t)
    with SafetensorsFile(path) as f:
        assert set(f.names()) == {"a", "b", "c"}
        for k in t:
            assert torch.equal(f.read(k), t[k])
    # the plain reader takes floating types only
    write_safetensors(path, {k: v for k, v in t.items() if k != "c"})
    plain = plain_gpt2.read_safetensors(path)
    assert np.array_equal(plain["a"], t["a"].double().numpy())
    assert np.array_equal(plain["b"], t["b"].double().numpy())


def _raw_file(path, header: dict, payload: bytes, header_len=None):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob) if header_len is None else header_len))
        f.write(blob)
        f.write(payload)


@pytest.mark.parametrize("header,payload,match", [
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 12]}}, b"\0" * 12, "needs 8"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, "outside the payload"),
    ({"a": {"dtype": "F99", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8, "unknown dtype"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [8, 0]}}, b"\0" * 8, "outside the payload|data_offsets"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0]}}, b"\0" * 8, "pair"),
])
def test_reader_rejects_bad_files(tmp_path, header, payload, match):
    path = str(tmp_path / "bad.safetensors")
    _raw_file(path, header, payload)
    with pytest.raises(SafetensorsError, match=match):
        SafetensorsFile(path)


def test_reader_rejects_bad_header_length(tmp_path):
    path = str(tmp_path / "bad.safetensors")
    _raw_file(path, {}, b"", header_len=10 ** 9)
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(path)
    with open(path, "wb") as f:
        f.write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(path)


def test_random_model_loads_and_is_reproducible(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_A, seed=5)
    b = write_random_model(str(tmp_path / "b"), TINY_A, seed=5)
    c = write_random_model(str(tmp_path / "c"), TINY_A, seed=6)
    wa, wb, wc = (plain_gpt2.read_safetensors(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert all(np.array_equal(wa[k], wb[k]) for k in wa)
    assert not np.array_equal(wa["wte.weight"], wc["wte.weight"])
    # same-shaped tensors differ, norm weights sit around one, residual projections are narrower
    assert not np.array_equal(wa["h.0.ln_1.bias"], wa["h.1.ln_1.bias"])
    assert abs(wa["h.0.ln_1.weight"].mean() - 1.0) < 0.02
    assert wa["h.0.mlp.c_proj.weight"].std() < 0.7 * wa["h.0.mlp.c_fc.weight"].std()
    with open(os.path.join(a, "config.json")) as f:
        assert json.load(f)["n_inner"] == 256
    plan = Gpt2Config.from_json(TINY_A).plan()
    loaded = load_weights(a, collect_tensor_specs(plan), torch.bfloat16, "cpu", ignored=plan.ignored_tensors)
    assert loaded["h.0.attn.c_attn.weight"].shape == (192, 64)          # transposed to [out, in]
    assert loaded["h.0.attn.c_attn.weight"].dtype == torch.bfloat16
    assert loaded["h.0.attn.c_attn.bias"].dtype == torch.float32        # vectors are kept in 32-bit
    stored = wa["h.0.attn.c_attn.weight"]
    assert np.array_equal(loaded["h.0.attn.c_attn.weight"].double().numpy(), stored.T)


def test_float32_file_stays_float32_on_the_32_bit_path(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, seed=1, store_dtype="float32")
    plan = Gpt2Config.from_json(TINY_B).plan()
    specs = collect_tensor_specs(plan)
    w32 = load_weights(d, specs, torch.float32, "cpu", ignored=plan.ignored_tensors)
    raw = plain_gpt2.read_safetensors(os.path.join(d, "model.safetensors"), dtype=np.float32)
    assert w32["wte.weight"].dtype == torch.float32
    assert np.array_equal(w32["wte.weight"].numpy(), raw["wte.weight"])          # not a bit is lost


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=2)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.read(n) for n in f.names()}
    del tensors["h.1.mlp.c_fc.bias"]
    del tensors["ln_f.weight"]
    tensors["h.0.attn.c_proj.weight"] = torch.zeros(64, 65, dtype=torch.bfloat16)
    tensors["h.7.extra.weight"] = torch.zeros(2)
    tensors["h.0.attn.bias"] = torch.zeros(1, 1, 4, 4)           # the checkpoint's mask buffer: ignored
    tensors["lm_head.weight"] = torch.zeros(512, 64)             # a tied copy: ignored
    write_safetensors(path, tensors)
    plan = Gpt2Config.from_json(TINY_A).plan()
    with pytest.raises(WeightError) as e:
        load_weights(d, collect_tensor_specs(plan), torch.float32, "cpu", ignored=plan.ignored_tensors)
    err = e.value
    assert err.missing == ["h.1.mlp.c_fc.bias", "ln_f.weight"]
    assert err.unexpected == ["h.7.extra.weight"]
    assert err.wrong_shape == [("h.0.attn.c_proj.weight", (64, 65), (64, 64))]
    text = str(err)
    assert "missing (2)" in text and "unexpected (1)" in text and "wrong shape (1)" in text


def test_prefixed_names_are_found(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=2)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {"transformer." + n: f.read(n) for n in f.names()}
    write_safetensors(path, tensors)
    plan = Gpt2Config.from_json(TINY_A).plan()
    w = load_weights(d, collect_tensor_specs(plan), torch.float32, "cpu", ignored=plan.ignored_tensors,
                     prefixes=("", "transformer."))
    assert "wte.weight" in w and len(w) == len(tensors)
    # the usual layout of such a checkpoint: layers under the prefix, the tied output copy beside them
    tensors["lm_head.weight"] = torch.zeros(512, 64)
    write_safetensors(path, tensors)
    w = load_weights(d, collect_tensor_specs(plan), torch.float32, "cpu", ignored=plan.ignored_tensors,
                     prefixes=("", "transformer."))
    assert "lm_head.weight" not in w and len(w) == len(tensors) - 1


def test_bias_modes_of_a_part(tmp_path):
    """A part's ``bias`` parameter: true wants the vector in the file, "if_present" takes it when it
    is there, false never reads it (a file that holds it anyway has an unexpected tensor)."""
    import dataclasses
    d = write_random_model(str(tmp_path / "m"), TINY_A, seed=2)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.read(n) for n in f.names()}
    del tensors["h.0.mlp.c_fc.bias"]
    write_safetensors(path, tensors)
    plan = Gpt2Config.from_json(TINY_A).plan()

    def with_bias(mode):
        layers = list(plan.layers)
        ff = layers[0].feed_forward
        layers[0] = dataclasses.replace(layers[0], feed_forward=dataclasses.replace(ff, params=dict(ff.params, bias=mode)))
        return dataclasses.replace(plan, layers=tuple(layers))

    with pytest.raises(WeightError) as e:
        load_weights(d, collect_tensor_specs(with_bias(True)), torch.float32, "cpu", ignored=plan.ignored_tensors)
    assert e.value.missing == ["h.0.mlp.c_fc.bias"]
    w = load_weights(d, collect_tensor_specs(with_bias("if_present")), torch.float32, "cpu",
                     ignored=plan.ignored_tensors)
    assert "h.0.mlp.c_fc.bias" not in w and "h.0.mlp.c_proj.bias" in w
    with pytest.raises(WeightError) as e:
        load_weights(d, collect_tensor_specs(with_bias(False)), torch.float32, "cpu", ignored=plan.ignored_tensors)
    assert e.value.unexpected == ["h.0.mlp.c_proj.bias"] and not e.value.missing
