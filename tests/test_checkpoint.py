"""The checkpoint loader (cohere-inference_b200/checkpoint.py) on the CPU: the rename table against the names
transformers' own save_pretrained writes (tests/golden/checkpoint_names.json, made by make_checkpoint_names.py), a
checkpoint directory written here in that naming (single file and sharded, fp32 and bf16) read back bit for bit, and
the errors a damaged directory must raise. The GPU half (a decoder built from such a directory equals the one built
from the module) is in test_gpu_decoder.py."""

import json
import os
import struct

import numpy as np
import pytest
import torch

from cohere_inference_b200 import checkpoint as ck
from cohere_inference_b200 import synthetic_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "checkpoint_names.json")
CODES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int64: "I64"}


def write_safetensors(path: str, tensors: dict) -> None:
    """The published layout: u64 header length, JSON header, raw little-endian data (8-byte aligned start)."""
    header, blobs, at = {"__metadata__": {"format": "pt"}}, [], 0
    for name, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = dict(dtype=CODES[t.dtype], shape=list(t.shape), data_offsets=[at, at + len(raw)])
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))


def original_names() -> dict:
    """module name -> the name a published checkpoint gives it, for a 2-layer decoder, from the golden list"""
    with open(GOLDEN) as f:
        return {v["module"]: k for k, v in json.load(f)["decoder"].items()}


def tiny_model(dtype=torch.float32):
    return synthetic_model(5, heads=4, head_dim=16, act="relu", layers=2, hidden=64, ffn=128, vocab=96, max_pos=32,
                           bias_std=0.05, dtype=dtype)


def write_checkpoint(d, model, *, names=None, shards=1, encoder_hidden=64) -> None:
    c = model.config
    cfg = dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, num_hidden_layers=c.num_hidden_layers,
               num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
               head_dim=c.head_dim, intermediate_size=c.intermediate_size, hidden_act=c.hidden_act,
               max_position_embeddings=c.max_position_embeddings, pad_token_id=2, eos_token_id=3, bos_token_id=4,
               model_type="cohere_asr", encoder_config=dict(hidden_size=encoder_hidden, subsampling_factor=8))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    state = {(names[k] if names else k): v.detach() for k, v in model.state_dict().items()}
    # what a real file is mostly made of: encoder tensors, which the loader must pass over
    state["model.encoder.layers.0.self_attn.linear_q.weight"] = torch.randn(8, 8)
    state["model.encoder.layers.0.norm_out.layer_norm_1.weight"] = torch.randn(8)  # a decoder-like fragment in its name
    state["model.encoder.pre_encode.out.bias"] = torch.randn(8)
    keys = list(state)
    if shards == 1:
        write_safetensors(os.path.join(d, "model.safetensors"), state)
        return
    weight_map = {}
    for i in range(shards):
        fn = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        part = {k: state[k] for k in keys[i::shards]}
        write_safetensors(os.path.join(d, fn), part)
        weight_map.update({k: fn for k in part})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump(dict(metadata={}, weight_map=weight_map), f)


def test_rename_table_matches_what_transformers_writes():
    with open(GOLDEN) as f:
        g = json.load(f)
    assert len(g["decoder"]) == 62  # 2 layers x 26 + 10
    for name, want in g["decoder"].items():
        assert ck.module_name(name) == want["module"], name
        assert ck.module_name(want["module"]) == want["module"]  # files written with the module names load too
    for name in g["encoder_examples"]:
        assert ck.module_name(name) is None, name
    # every key read_config looks up is one save_pretrained writes
    assert {"vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
            "intermediate_size", "hidden_act", "max_position_embeddings", "pad_token_id", "eos_token_id",
            "bos_token_id", "encoder_config"} <= set(g["config_keys"])
    assert {"hidden_size", "subsampling_factor"} <= set(g["encoder_config_keys"])


@pytest.mark.parametrize("style,shards,dtype", [("original", 1, torch.float32), ("original", 3, torch.bfloat16),
                                                ("module", 1, torch.bfloat16), ("module", 2, torch.float32)])
def test_directory_round_trip_is_bit_exact(tmp_path, style, shards, dtype):
    model = tiny_model(dtype)
    write_checkpoint(str(tmp_path), model, names=original_names() if style == "original" else None, shards=shards)
    got = ck.load_decoder(str(tmp_path))
    a, b = got.state_dict(), model.state_dict()
    assert a.keys() == b.keys()
    for k in a:
        assert a[k].dtype == dtype and torch.equal(a[k], b[k]), k
    c = got.config
    assert (c.num_attention_heads, c.head_dim, c.hidden_act, c.num_hidden_layers) == (4, 16, "relu", 2)
    assert int(got.model.encoder._get_subsampling_output_length(torch.tensor([3001]))) == 376
    # conversion on load: what the reference does with dtype=torch.bfloat16
    conv = ck.load_decoder(str(tmp_path), torch.bfloat16).state_dict()
    assert all(conv[k].dtype == torch.bfloat16 and torch.equal(conv[k], b[k].to(torch.bfloat16)) for k in b)


def test_wider_encoder_projection(tmp_path):
    """The real model projects 1280-wide encoder frames to the decoder's width: the width comes from encoder_config."""
    model = tiny_model()
    model.model.decoder.proj = torch.nn.Linear(80, 64)
    write_checkpoint(str(tmp_path), model, names=original_names(), encoder_hidden=80)
    got = ck.load_decoder(str(tmp_path))
    assert got.config.encoder_hidden_size == 80
    assert torch.equal(got.model.decoder.proj.weight, model.model.decoder.proj.weight)


def test_damaged_directories_raise(tmp_path):
    model, names = tiny_model(), original_names()
    d = str(tmp_path)
    write_checkpoint(d, model, names=names)
    path = os.path.join(d, "model.safetensors")
    with ck.SafetensorsFile(path) as sf:
        state = {n: sf.tensor(n) for n in sf.names()}
    # a decoder tensor missing
    short = dict(state)
    del short["model.transf_decoder._decoder.layers.1.third_sub_layer.dense_out.bias"]
    write_safetensors(path, short)
    with pytest.raises(KeyError, match="missing"):
        ck.load_decoder(d)
    # a shape that contradicts the config
    bad = dict(state)
    bad["log_softmax.mlp.layer0.weight"] = torch.zeros(95, 64)
    write_safetensors(path, bad)
    with pytest.raises(ValueError, match="shape"):
        ck.load_decoder(d)
    # a decoder tensor the decoder has no place for
    extra = dict(state)
    extra["model.transf_decoder._decoder.layers.2.layer_norm_1.weight"] = torch.zeros(64)
    write_safetensors(path, extra)
    with pytest.raises(KeyError, match="no place"):
        ck.load_decoder(d)
    # a header that lies about the file
    write_safetensors(path, state)
    blob = open(path, "rb").read()
    with open(path, "wb") as f:
        f.write(blob[:-16])
    with pytest.raises(ValueError, match="claims|fit"):
        ck.load_decoder(d)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="header length"):
        ck.load_decoder(d)
    os.remove(path)
    with pytest.raises(FileNotFoundError):
        ck.load_decoder(d)


def test_only_the_decoder_shards_are_opened(tmp_path):
    model = tiny_model()
    d = str(tmp_path)
    write_checkpoint(d, model, names=original_names(), shards=2)
    # a third shard of encoder tensors only, listed in the index, that does not exist on disk: never opened
    index = os.path.join(d, "model.safetensors.index.json")
    with open(index) as f:
        idx = json.load(f)
    idx["weight_map"]["model.encoder.layers.7.feed_forward1.linear1.weight"] = "model-encoder-only.safetensors"
    with open(index, "w") as f:
        json.dump(idx, f)
    got = ck.load_decoder(d)
    assert all(torch.equal(v, model.state_dict()[k]) for k, v in got.state_dict().items())
    assert np.isfinite(got.proj_out.weight.float().numpy()).all()
