"""The safetensors reader/writer and the strict by-name loader (on the CPU: loading needs
no kernel)."""

from __future__ import annotations

import pytest
import torch

from tiny_configs import ALL, SEEDS

from emberserve_b200.registry import build_decoder
from emberserve_b200.weights.loader import WeightsError, load_weights, random_checkpoint, write_random_model
from emberserve_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors


def test_own_reader_and_the_safetensors_package_agree(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).view(2, 3), "d": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "mine.safetensors", t, metadata={"k": "v"})
    with safe_open(str(tmp_path / "mine.safetensors"), framework="pt") as f:
        assert set(f.keys()) == set(t)
        for k in t:
            assert torch.equal(f.get_tensor(k), t[k])
    save_file(t, str(tmp_path / "theirs.safetensors"))
    mine = SafetensorsFile(tmp_path / "theirs.safetensors")
    for k in t:
        assert torch.equal(mine.get(k), t[k]) and mine.tensors[k].dtype == t[k].dtype


def test_truncated_file_is_refused(tmp_path):
    write_safetensors(tmp_path / "x.safetensors", {"a": torch.randn(100)})
    raw = (tmp_path / "x.safetensors").read_bytes()
    (tmp_path / "x.safetensors").write_bytes(raw[:-40])
    with pytest.raises(SafetensorsError, match="spans bytes"):
        SafetensorsFile(tmp_path / "x.safetensors")


@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_round_trip(tmp_path, name, dtype):
    cfg = ALL[name]
    folder = write_random_model(cfg, tmp_path / name, SEEDS[name])
    dec = build_decoder(cfg)
    params = load_weights(dec, folder, "cpu", dtype)
    src = random_checkpoint(build_decoder(cfg), SEEDS[name])
    assert all(p.dtype == dtype for p in params.values())
    q = cfg.num_attention_heads * cfg.head_dim
    kv = cfg.num_key_value_heads * cfg.head_dim
    w = params["layers.1.mixer.wqkv"]
    assert torch.equal(w[:q], src["model.layers.1.self_attn.q_proj.weight"].to(dtype))
    assert torch.equal(w[q:q + kv], src["model.layers.1.self_attn.k_proj.weight"].to(dtype))
    assert torch.equal(w[q + kv:], src["model.layers.1.self_attn.v_proj.weight"].to(dtype))
    i = cfg.intermediate_size
    assert torch.equal(params["layers.0.ffn.wgu"][i:], src["model.layers.0.mlp.up_proj.weight"].to(dtype))
    assert (dec.head is dec.embed) == cfg.tie_word_embeddings
    assert torch.equal(params["final_norm.weight"], torch.ones(cfg.hidden_size, dtype=dtype))


def test_32bit_tensors_stay_32bit_and_tables_are_int32(tmp_path):
    cfg = ALL["tiny_b"]
    t = random_checkpoint(build_decoder(cfg), 1)
    t["model.norm.weight"] = t["model.norm.weight"].float() * 1.0001  # stored in 32 bits
    t["model.layers.0.self_attn.q_proj.bias"] = t["model.layers.0.self_attn.q_proj.bias"].float()
    cfg.save(tmp_path)
    write_safetensors(tmp_path / "model.safetensors", t)
    params = load_weights(build_decoder(cfg), tmp_path, "cpu", torch.bfloat16)
    assert params["final_norm.weight"].dtype == torch.float32
    assert params["layers.0.mixer.bqkv"].dtype == torch.float32  # one 32-bit source keeps it wide
    assert params["layers.1.mixer.bqkv"].dtype == torch.bfloat16
    assert params["embed"].dtype == torch.bfloat16


def test_one_error_lists_everything(tmp_path):
    cfg = ALL["tiny_b"]
    t = random_checkpoint(build_decoder(cfg), 1)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["lm_head.weight"]
    t["model.layers.9.bogus.weight"] = torch.zeros(2)
    t["model.rotary_emb.inv_freq"] = torch.zeros(16)  # tolerated
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(5, 5)
    t["model.norm.weight"] = torch.zeros(cfg.hidden_size + 1)
    cfg.save(tmp_path)
    write_safetensors(tmp_path / "model.safetensors", t)
    with pytest.raises(WeightsError) as e:
        load_weights(build_decoder(cfg), tmp_path, "cpu", torch.float32)
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.9.bogus.weight"]
    assert {m[0] for m in err.mismatched} == {"model.layers.0.self_attn.k_proj.weight", "model.norm.weight"}
    for word in ("missing", "unexpected", "wrong shapes", "bogus", "(5, 5)"):
        assert word in str(err)


def test_tied_checkpoint_may_carry_the_head_and_shards_are_merged(tmp_path):
    cfg = ALL["tiny_a"]
    t = random_checkpoint(build_decoder(cfg), 0)
    names = sorted(t)
    cfg.save(tmp_path)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {k: t[k] for k in names[::2]})
    second = {k: t[k] for k in names[1::2]}
    second["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", second)
    params = load_weights(build_decoder(cfg), tmp_path, "cpu", torch.float32)
    assert torch.equal(params["embed"], t["model.embed_tokens.weight"].float())
    write_safetensors(tmp_path / "model-00003-of-00003.safetensors", {names[0]: t[names[0]]})
    with pytest.raises(WeightsError, match="more than one file"):
        load_weights(build_decoder(cfg), tmp_path, "cpu", torch.float32)


def test_no_files(tmp_path):
    ALL["tiny_a"].save(tmp_path)
    with pytest.raises(FileNotFoundError):
        load_weights(build_decoder(ALL["tiny_a"]), tmp_path, "cpu", torch.float32)


def test_seed_and_deviation(tmp_path):
    cfg = ALL["tiny_b"]
    a = random_checkpoint(build_decoder(cfg), 5, store_dtype=torch.float32)
    b = random_checkpoint(build_decoder(cfg), 5, store_dtype=torch.float32)
    c = random_checkpoint(build_decoder(cfg), 6, store_dtype=torch.float32, std=0.5, bias_std=0.1)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert abs(float(a["model.embed_tokens.weight"].std()) - 0.02) < 2e-3
    assert abs(float(c["model.embed_tokens.weight"].std()) - 0.5) < 5e-2
    assert abs(float(c["model.layers.0.self_attn.q_proj.bias"].std()) - 0.1) < 3e-2
    assert torch.equal(a["model.layers.2.input_layernorm.weight"], torch.ones(cfg.hidden_size))


@pytest.mark.parametrize("name", list(ALL))
def test_export_is_the_inverse_of_the_load(tmp_path, name):
    """A loaded model written out again carries the checkpoint's names and bits (the fused
    projections cut back into q / k / v and gate / up, a tied head written once) and loads
    back into equal parameters."""
    from emberserve_b200.weights.loader import export_checkpoint, save_model

    folder = write_random_model(ALL[name], tmp_path / "src", SEEDS[name])
    original = SafetensorsFile(folder / "model.safetensors")
    decoder = build_decoder(ALL[name])
    params = load_weights(decoder, folder, "cpu", torch.bfloat16)
    exported = export_checkpoint(decoder)
    assert set(exported) == set(original.tensors)
    for key, tensor in exported.items():
        assert torch.equal(tensor, original.get(key)), key
    copy = save_model(decoder, ALL[name], tmp_path / "copy")
    again = load_weights(build_decoder(ALL[name]), copy, "cpu", torch.bfloat16)
    assert set(again) == set(params) and all(torch.equal(again[k], params[k]) for k in params)
