import json
import struct

import numpy as np
import pytest
import torch

import plain_gpt2
import tiny_models
from ayaka_py_b200.config import GPT2Config
from ayaka_py_b200.engine.loading import load_model, random_model
from ayaka_py_b200.weights import (CheckpointCorruptError, SafetensorsFile, UnsupportedWeightFormatError,
                                   WeightMismatchError, write_random_model, write_safetensors)


def test_loads_by_name_with_conv1d_layout(model_folders):
    folder, cfg, weights = model_folders["B"]
    config, model = load_model(folder, "float32", "cpu")
    attn = model.blocks[1].mixer
    assert attn.qkv_weight.shape == (288, 96) and attn.qkv_weight.dtype == torch.float32
    assert np.array_equal(attn.qkv_weight.numpy(), weights["transformer.h.1.attn.c_attn.weight"].T)
    assert np.array_equal(model.blocks[2].ffn.down_weight.numpy(), weights["transformer.h.2.mlp.c_proj.weight"].T)
    assert model.head.weight.data_ptr() == model.embedding.weight.data_ptr()      # tied: one tensor
    assert model.final_norm.weight.dtype == torch.float32
    _, bf = load_model(folder, "bfloat16", "cpu")
    assert bf.blocks[0].ffn.up_weight.dtype == torch.bfloat16
    assert bf.blocks[0].ffn.up_bias.dtype == torch.float32 and bf.blocks[0].norm1.weight.dtype == torch.float32
    assert np.array_equal(bf.embedding.weight.float().numpy(), weights["transformer.wte.weight"])


def _rewrite(folder, tmp_path, change):
    tensors = {k: torch.from_numpy(v.copy()) for k, v in
               plain_gpt2.read_safetensors(folder / "model.safetensors").items()}
    change(tensors)
    out = tmp_path / "changed"
    out.mkdir(parents=True)
    (out / "config.json").write_text((folder / "config.json").read_text())
    write_safetensors(out / "model.safetensors", tensors)
    return out


def test_one_error_lists_everything(model_folders, tmp_path):
    folder, cfg, _ = model_folders["A"]

    def change(t):
        del t["transformer.h.0.ln_1.bias"]
        del t["transformer.wpe.weight"]
        t["transformer.h.7.extra"] = torch.zeros(3)
        t["transformer.h.1.mlp.c_fc.weight"] = torch.zeros(256, 64)     # [out, in] instead of [in, out]
        t["transformer.ln_f.weight"] = torch.zeros(64, dtype=torch.int32)

    with pytest.raises(WeightMismatchError) as err:
        load_model(_rewrite(folder, tmp_path, change), "float32", "cpu")
    e = err.value
    assert e.missing == ["transformer.h.0.ln_1.bias", "transformer.wpe.weight"]
    assert e.unexpected == ["transformer.h.7.extra"]
    assert len(e.wrong) == 2 and "(256, 64)" in e.wrong[0] + e.wrong[1]
    text = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape or dtype (2)", "transformer.h.7.extra"):
        assert needle in text


def test_name_rules(model_folders, tmp_path):
    folder, cfg, weights = model_folders["A"]

    def change(t):
        for name in list(t):
            t[name.removeprefix("transformer.")] = t.pop(name)         # hub exports drop the prefix
        t["h.0.attn.bias"] = torch.ones(1, 1, 8, 8)                    # legacy mask buffers
        t["h.0.attn.masked_bias"] = torch.tensor(-1e4)
        t["lm_head.weight"] = t["wte.weight"].clone()                  # shipped though tied

    _, model = load_model(_rewrite(folder, tmp_path, change), "float32", "cpu")
    assert np.array_equal(model.position.weight.numpy(), weights["transformer.wpe.weight"])


def test_untied_head_needs_its_tensor(model_folders, tmp_path):
    folder, cfg, _ = model_folders["A"]
    out = _rewrite(folder, tmp_path, lambda t: None)
    (out / "config.json").write_text(json.dumps({**cfg, "tie_word_embeddings": False}))
    with pytest.raises(WeightMismatchError) as err:
        load_model(out, "float32", "cpu")
    assert err.value.missing == ["lm_head.weight"]


@pytest.mark.parametrize("damage", ["short", "header_past_end", "not_json", "duplicate", "dtype", "offsets",
                                    "bytes", "overlap"])
def test_corrupt_files(tmp_path, damage):
    path = tmp_path / "model.safetensors"
    header = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
              "b": {"dtype": "F32", "shape": [1], "data_offsets": [8, 12]}}
    payload = b"\0" * 12
    text = json.dumps(header)
    if damage == "short":
        path.write_bytes(b"\1\2\3")
    else:
        if damage == "not_json":
            text = "{" + text
        if damage == "duplicate":
            text = '{"a": {"dtype":"F32","shape":[1],"data_offsets":[0,4]}, "a": {"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
        if damage == "dtype":
            text = text.replace('"F32", "shape": [2]', '"F7", "shape": [2]')
        if damage == "offsets":
            text = text.replace("[8, 12]", "[8, 16]")
        if damage == "bytes":
            text = text.replace('"shape": [2]', '"shape": [3]')
        if damage == "overlap":
            text = text.replace("[8, 12]", "[4, 8]")
        raw = text.encode()
        length = len(raw) + (10 ** 6 if damage == "header_past_end" else 0)
        path.write_bytes(struct.pack("<Q", length) + raw + payload)
    with pytest.raises(CheckpointCorruptError):
        SafetensorsFile(path)


@pytest.mark.parametrize("token", ["F4", "I4", "U4", "F8_E4M3", "F8_E5M2"])
def test_packed_and_quantized_dtypes_are_refused_as_unsupported(tmp_path, token):
    """``model_loader/st.py:98-131``: a known sub-byte or 8-bit float dtype is not a corrupt file."""
    path = tmp_path / "model.safetensors"
    raw = json.dumps({"w": {"dtype": token, "shape": [4], "data_offsets": [0, 4]}}).encode()
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + b"\0" * 4)
    with pytest.raises(UnsupportedWeightFormatError) as err:
        SafetensorsFile(path)
    assert token in str(err.value) and not isinstance(err.value, CheckpointCorruptError)


def test_dtype_rule_narrowing_and_widening(model_folders, tmp_path):
    """``model_loader/validate.py:83-95``: float32 -> bfloat16 is the one narrowing; float16 read
    as bfloat16 and float64 into anything are listed as wrong, together, in the one error."""
    folder, cfg, weights = model_folders["A"]

    def change(t):
        t["transformer.h.0.mlp.c_fc.weight"] = t["transformer.h.0.mlp.c_fc.weight"].to(torch.float16)
        t["transformer.h.1.attn.c_proj.weight"] = t["transformer.h.1.attn.c_proj.weight"].to(torch.float64)
        t["transformer.ln_f.bias"] = t["transformer.ln_f.bias"].to(torch.float64)

    changed = _rewrite(folder, tmp_path, change)
    with pytest.raises(WeightMismatchError) as err:
        load_model(changed, "bfloat16", "cpu")
    wrong = "\n".join(err.value.wrong)
    assert len(err.value.wrong) == 3 and not err.value.missing and not err.value.unexpected
    assert "c_fc.weight: dtype torch.float16 cannot feed torch.bfloat16" in wrong
    assert "attn.c_proj.weight: dtype torch.float64" in wrong and "ln_f.bias: dtype torch.float64" in wrong
    with pytest.raises(WeightMismatchError) as err:              # 32-bit engine: float16 widens, float64 does not
        load_model(changed, "float32", "cpu")
    assert len(err.value.wrong) == 2 and all("float64" in w for w in err.value.wrong)
    # float32 stored -> bfloat16 engine (narrowing) and bfloat16 stored -> float32 engine (widening) load
    _, narrow = load_model(folder, "bfloat16", "cpu")
    assert narrow.blocks[0].ffn.up_weight.dtype == torch.bfloat16
    bf = _rewrite(folder, tmp_path / "bf", lambda t: t.update(
        {k: v.to(torch.bfloat16) for k, v in t.items() if k.endswith("c_fc.weight")}))
    _, wide = load_model(bf, "float32", "cpu")
    assert wide.blocks[0].ffn.up_weight.dtype == torch.float32


def _shard(folder, out, split, index_names=None):
    """Writes ``folder``'s tensors as two shards with an index; ``index_names`` limits what the index lists."""
    tensors = {k: torch.from_numpy(v.copy()) for k, v in
               plain_gpt2.read_safetensors(folder / "model.safetensors").items()}
    names = sorted(tensors)
    parts = {"model-00001-of-00002.safetensors": names[:split], "model-00002-of-00002.safetensors": names[split:]}
    out.mkdir(parents=True)
    (out / "config.json").write_text((folder / "config.json").read_text())
    weight_map = {}
    for shard, members in parts.items():
        write_safetensors(out / shard, {n: tensors[n] for n in members})
        weight_map.update({n: shard for n in members if index_names is None or n in index_names})
    (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    return out, tensors


def test_sharded_folder_loads_and_reports_what_the_index_omits(model_folders, tmp_path):
    folder, cfg, weights = model_folders["B"]
    out, tensors = _shard(folder, tmp_path / "sharded", split=11)
    _, model = load_model(out, "float32", "cpu")
    assert np.array_equal(model.blocks[2].ffn.down_weight.numpy(), weights["transformer.h.2.mlp.c_proj.weight"].T)
    assert np.array_equal(model.embedding.weight.numpy(), weights["transformer.wte.weight"])
    # a shard holds a tensor that the index does not list and the model does not want: unexpected, not ignored
    extra = tmp_path / "extra"
    listed = set(tensors)
    out2, _ = _shard(folder, extra, split=11, index_names=listed)
    first = extra / "model-00001-of-00002.safetensors"
    kept = {k: torch.from_numpy(v.copy()) for k, v in plain_gpt2.read_safetensors(first).items()}
    kept["transformer.h.9.stray.weight"] = torch.zeros(2, 2)
    write_safetensors(first, kept)
    with pytest.raises(WeightMismatchError) as err:
        load_model(out2, "float32", "cpu")
    assert err.value.unexpected == ["transformer.h.9.stray.weight"] and not err.value.missing
    # a tensor the model wants lies in a shard although the index forgot it: it is found
    partial = tmp_path / "partial"
    out3, _ = _shard(folder, partial, split=11, index_names=listed - {"transformer.ln_f.weight"})
    _, model3 = load_model(out3, "float32", "cpu")
    assert np.array_equal(model3.final_norm.weight.numpy(), weights["transformer.ln_f.weight"])


def test_untied_head_is_loaded_and_used(model_folders, tmp_path):
    folder, cfg, weights = model_folders["A"]
    head = np.random.RandomState(3).standard_normal(weights["transformer.wte.weight"].shape).astype(np.float32) * 0.05

    out = _rewrite(folder, tmp_path, lambda t: t.update({"lm_head.weight": torch.from_numpy(head.copy())}))
    (out / "config.json").write_text(json.dumps({**cfg, "tie_word_embeddings": False}))
    _, model = load_model(out, "float32", "cpu")
    assert model.head.weight.data_ptr() != model.embedding.weight.data_ptr()
    assert np.array_equal(model.head.weight.numpy(), head)
    config, tensors = plain_gpt2.read_model_folder(out)
    logits = plain_gpt2.forward(config, tensors, [5, 6, 7])
    tied = plain_gpt2.forward(*plain_gpt2.read_model_folder(folder), [5, 6, 7])
    assert np.abs(logits - tied).max() > 1e-3                    # the plain implementation uses the head it is given


def test_random_mode_writes_a_loadable_folder(tmp_path):
    cfg = GPT2Config.from_dict(tiny_models.TINY_B)
    folder = write_random_model(tmp_path / "m", cfg, seed=7)
    document = json.loads((folder / "config.json").read_text())
    assert document["architectures"] == ["GPT2LMHeadModel"] and document["n_inner"] == 320
    config, tensors = plain_gpt2.read_model_folder(folder)
    assert tensors["transformer.h.0.attn.c_attn.weight"].shape == (96, 288)        # Conv1D layout
    again = write_random_model(tmp_path / "m2", cfg, seed=7)
    assert (again / "model.safetensors").read_bytes() == (folder / "model.safetensors").read_bytes()
    other = write_random_model(tmp_path / "m3", cfg, seed=8)
    assert (other / "model.safetensors").read_bytes() != (folder / "model.safetensors").read_bytes()
    w = tensors["transformer.h.2.mlp.c_proj.weight"]
    assert abs(w.std() - 0.02 / np.sqrt(6)) < 1e-3
    assert abs(tensors["transformer.h.1.ln_1.weight"].mean() - 1.0) < 0.03
    with SafetensorsFile(folder / "model.safetensors") as f:
        assert f.entries["transformer.wte.weight"].dtype == "BF16"
        assert f.entries["transformer.ln_f.bias"].dtype == "F32"
    _, model = load_model(folder, "bfloat16", "cpu")
    direct = random_model(cfg, 7, "bfloat16", "cpu")
    assert torch.equal(model.blocks[1].mixer.out_weight, direct.blocks[1].mixer.out_weight)
    logits = plain_gpt2.forward(config, tensors, [1, 2, 3])
    assert logits.shape == (3, 1000) and np.isfinite(logits).all()
