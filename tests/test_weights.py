"""Safetensors reading/writing and the loader's errors (no GPU: buffers live on the CPU)."""

import struct

import pytest
import torch

import plain_model
from dryft_flash_infer_b200 import models  # noqa: F401
from dryft_flash_infer_b200.config import architecture_named, config_from_dict, load_config
from dryft_flash_infer_b200.engine.model import DecoderModel
from dryft_flash_infer_b200.weights import (ModelFiles, SafetensorsError, SafetensorsFile, WeightError,
                                            load_weights, random_tensor, write_random_model, write_safetensors)


def _model(cfg_dict, dtype=torch.float32):
    cfg = config_from_dict(cfg_dict)
    model = DecoderModel(architecture_named(cfg.architecture).build(cfg))
    model.allocate(dtype, "cpu")
    return model


def _folder(tmp_path, cfg_dict, weights):
    config_from_dict(cfg_dict).save(tmp_path)
    write_safetensors(tmp_path / "model.safetensors", weights.items())
    return tmp_path


def test_safetensors_round_trip(tmp_path):
    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
        "c": torch.arange(6, dtype=torch.int32).view(2, 3), "d": torch.randn(2, 2).to(torch.float16),
        "empty": torch.zeros(0, 4),
    }
    write_safetensors(tmp_path / "x.safetensors", tensors.items(), metadata={"k": "v"})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert set(f.names()) == set(tensors) and f.metadata == {"k": "v"}
    for name, t in tensors.items():
        assert f.info(name) == (t.dtype, tuple(t.shape))
        assert torch.equal(f.tensor(name), t)
    # the layout is the published one: 8-byte length, JSON, data
    raw = (tmp_path / "x.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    assert raw[8:8 + n].lstrip().startswith(b"{")


def test_truncated_and_broken_files(tmp_path):
    write_safetensors(tmp_path / "x.safetensors", {"a": torch.randn(64, 64)}.items())
    raw = (tmp_path / "x.safetensors").read_bytes()
    (tmp_path / "cut.safetensors").write_bytes(raw[:-100])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(tmp_path / "cut.safetensors")
    (tmp_path / "short.safetensors").write_bytes(raw[:5])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(tmp_path / "short.safetensors")
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        ModelFiles(tmp_path)


def test_loads_by_name_into_fused_buffers(tmp_path):
    cfg = plain_model.TINY_B
    w = plain_model.random_weights(cfg, 4)
    model = _model(cfg)
    load_weights(model, _folder(tmp_path, cfg, w))
    mixer = model.blocks[1].mixer
    p = "model.layers.1.self_attn."
    assert torch.equal(mixer.qkv, torch.cat([w[p + "q_proj.weight"], w[p + "k_proj.weight"], w[p + "v_proj.weight"]]))
    assert torch.equal(mixer.q_norm, w[p + "q_norm.weight"])
    ffn = model.blocks[2].feed_forward
    assert torch.equal(ffn.gate_up, torch.cat([w["model.layers.2.mlp.gate_proj.weight"],
                                               w["model.layers.2.mlp.up_proj.weight"]]))
    assert torch.equal(model.head, w["lm_head.weight"]) and model.head is not model.embedding
    assert torch.equal(model.final_norm.weight, w["model.norm.weight"])


def test_dtypes_kept(tmp_path):
    cfg = plain_model.TINY_A
    w = plain_model.random_weights(cfg, 4)
    stored = {k: (v if v.dim() == 1 else v.to(torch.bfloat16)) for k, v in w.items()}  # norms in float32
    model = _model(cfg, torch.bfloat16)
    load_weights(model, _folder(tmp_path, cfg, stored))
    assert model.blocks[0].mixer.qkv.dtype == torch.bfloat16
    assert model.embedding.dtype == torch.bfloat16 and model.head is model.embedding  # tied
    norm = model.blocks[0].mixer_norm.weight
    assert norm.dtype == torch.float32 and torch.equal(norm, w["model.layers.0.input_layernorm.weight"])
    # a bfloat16 file read by the float32 engine is widened exactly
    model32 = _model(cfg, torch.float32)
    load_weights(model32, tmp_path)
    assert torch.equal(model32.embedding, stored["model.embed_tokens.weight"].float())


def test_one_error_lists_everything_wrong(tmp_path):
    cfg = plain_model.TINY_B
    w = plain_model.random_weights(cfg, 4)
    del w["model.layers.0.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.9.extra.weight"] = torch.zeros(2)
    w["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(32, 96)
    w["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(16)
    with pytest.raises(WeightError) as info:
        load_weights(_model(cfg), _folder(tmp_path, cfg, w))
    err = info.value
    assert set(err.missing) == {"model.layers.0.mlp.up_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.1.self_attn.k_proj.weight",
                                                  "model.layers.2.self_attn.q_norm.weight"}
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "model.layers.9.extra.weight",
                  "is [32, 96], expected [64, 96]"):
        assert piece in text


def test_tied_model_ignores_a_stored_head_and_untied_needs_it(tmp_path):
    cfg = plain_model.TINY_A
    w = plain_model.random_weights(cfg, 4)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    load_weights(_model(cfg), _folder(tmp_path, cfg, w))
    cfg_b = plain_model.TINY_B
    w_b = plain_model.random_weights(cfg_b, 4)
    del w_b["lm_head.weight"]
    (tmp_path / "b").mkdir()
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(_model(cfg_b), _folder(tmp_path / "b", cfg_b, w_b))


def test_integer_tensor_in_a_float_place_is_refused(tmp_path):
    cfg = plain_model.TINY_A
    w = plain_model.random_weights(cfg, 4)
    w["model.norm.weight"] = torch.ones(64, dtype=torch.int32)
    with pytest.raises(WeightError, match="unsupported dtype"):
        load_weights(_model(cfg), _folder(tmp_path, cfg, w))


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    cfg = config_from_dict(plain_model.TINY_B)
    write_random_model(cfg, 7, tmp_path / "m", dtype=torch.bfloat16)
    assert load_config(tmp_path / "m") == config_from_dict({**plain_model.TINY_B, "torch_dtype": "bfloat16"})
    files = ModelFiles(tmp_path / "m")
    model = _model(plain_model.TINY_B)
    load_weights(model, tmp_path / "m")
    assert files.info("model.layers.0.mlp.gate_proj.weight") == (torch.bfloat16, (200, 96))
    # same seed, same values; another seed, other values; the statistics asked for
    write_random_model(cfg, 7, tmp_path / "again", dtype=torch.bfloat16)
    assert torch.equal(ModelFiles(tmp_path / "again").tensor("lm_head.weight"), files.tensor("lm_head.weight"))
    write_random_model(cfg, 8, tmp_path / "other", dtype=torch.bfloat16)
    assert not torch.equal(ModelFiles(tmp_path / "other").tensor("lm_head.weight"), files.tensor("lm_head.weight"))
    big = random_tensor("m", (400, 400), "matrix", 1)
    assert abs(float(big.std()) - 0.02) < 1e-3 and abs(float(big.mean())) < 1e-3
    norm = random_tensor("n", (4000,), "norm", 1)
    assert abs(float(norm.mean()) - 1.0) < 1e-3 and abs(float(norm.std()) - 0.01) < 1e-3


def _raw_file(path, header: bytes, data: bytes = b""):
    path.write_bytes(struct.pack("<Q", len(header)) + header + data)
    return path


def test_native_reader_parses_and_checks_the_header(tmp_path):
    # names with escapes, an unknown key, metadata, and a tensor read piece by piece
    values = torch.arange(12, dtype=torch.float32)
    header = (b'{"__metadata__": {"note": "a \\"quoted\\" word", "n": "1"}, '
              b'"w\\u00e9ight \\"x\\"\\n": {"dtype": "F32", "extra": [1, {"a": null}], "shape": [3, 4], "data_offsets": [0, 48]}}')
    f = SafetensorsFile(_raw_file(tmp_path / "ok.safetensors", header, values.numpy().tobytes()))
    name = 'wéight "x"\n'
    assert f.names() == [name] and f.metadata == {"note": 'a "quoted" word', "n": "1"}
    assert torch.equal(f.tensor(name), values.view(3, 4))
    piece = torch.empty(5)
    assert torch.equal(f.read_into(name, piece, first_element=6), values[6:11])
    for bad, message in (
        (b'{"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}', "spans 4 bytes, shape needs 8"),
        (b'{"a": {"dtype": "F33", "shape": [1], "data_offsets": [0, 4]}}', "unsupported dtype F33"),
        (b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}', "not valid JSON"),
        (b'{"a": {"dtype": "F32", "shape": [1]}}', "lacks dtype, shape or data_offsets"),
        (b'{"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}', "not a size"),
        (b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}', "truncated"),
    ):
        with pytest.raises(SafetensorsError, match=message):
            SafetensorsFile(_raw_file(tmp_path / "bad.safetensors", bad, b"\0" * 4))
