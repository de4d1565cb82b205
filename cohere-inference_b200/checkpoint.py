"""The decoder half of a Cohere Transcribe checkpoint directory, read without building the model.

The reference loads the whole model through transformers (`CohereAsrForConditionalGeneration.from_pretrained`,
server.py:264-267) and hands it to its StreamDecoder, which then reads only `model.model.decoder.*` and
`model.proj_out` (kernels/stream_decoder.py:73-99). The encoder is four fifths of the file and is not on the decoder's
path, so this loader maps the checkpoint's `*.safetensors` files, takes the ~70 decoder tensors by name and fills the
attribute tree StreamDecoder reads (synth.SyntheticCohereAsr); the encoder's bytes are never touched.

Tensor names: a published checkpoint keeps the names of the training framework
(`model.transf_decoder._decoder.layers.N.first_sub_layer.query_net.weight`, `log_softmax.mlp.layer0.weight`,
`model.encoder_decoder_proj.weight`, ...), which transformers renames on load and restores on `save_pretrained`;
files written with the module names themselves (`model.decoder.layers.N.self_attn.q_proj.weight`, `proj_out.weight`)
are accepted as well. The file format (8-byte little-endian header length, a JSON header of
name -> {dtype, shape, data_offsets}, then the raw little-endian data) is read here directly.
"""

from __future__ import annotations

import json
import mmap
import os
import re
import struct

import numpy as np
import torch

from .synth import DecoderConfig, SyntheticCohereAsr

# checkpoint name -> module name, applied in order (the renames transformers applies for this model family)
_RENAMES = (
    (r"^log_softmax\.mlp\.layer0\.", "proj_out."),
    (r"^model\.transf_decoder\._embedding\.position_embedding\.pos_enc$", "model.decoder.pos_emb.weight"),
    (r"^model\.transf_decoder\._embedding\.token_embedding\.", "model.decoder.embed_tokens."),
    (r"^model\.transf_decoder\._embedding\.layer_norm\.", "model.decoder.embedding_layernorm."),
    (r"^model\.transf_decoder\._decoder\.final_layer_norm\.", "model.decoder.norm."),
    (r"^model\.transf_decoder\._decoder\.layers\.", "model.decoder.layers."),
    (r"^model\.encoder_decoder_proj\.", "model.decoder.proj."),
    (r"\.first_sub_layer\.query_net\.", ".self_attn.q_proj."),
    (r"\.first_sub_layer\.key_net\.", ".self_attn.k_proj."),
    (r"\.first_sub_layer\.value_net\.", ".self_attn.v_proj."),
    (r"\.first_sub_layer\.out_projection\.", ".self_attn.o_proj."),
    (r"\.second_sub_layer\.query_net\.", ".encoder_attn.q_proj."),
    (r"\.second_sub_layer\.key_net\.", ".encoder_attn.k_proj."),
    (r"\.second_sub_layer\.value_net\.", ".encoder_attn.v_proj."),
    (r"\.second_sub_layer\.out_projection\.", ".encoder_attn.o_proj."),
    (r"\.third_sub_layer\.dense_in\.", ".mlp.fc1."),
    (r"\.third_sub_layer\.dense_out\.", ".mlp.fc2."),
    (r"\.layer_norm_1\.", ".input_layernorm."),
    (r"\.layer_norm_2\.", ".post_attention_layernorm."),
    (r"\.layer_norm_3\.", ".final_layernorm."),
)
_RENAMES = tuple((re.compile(a), b) for a, b in _RENAMES)

_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool}


def module_name(name: str) -> str | None:
    """The decoder-path module name of a checkpoint tensor, or None for a tensor that is not on the path (encoder)."""
    for pat, rep in _RENAMES:
        name = pat.sub(rep, name)
    return name if name.startswith(("model.decoder.", "proj_out.")) else None


class SafetensorsFile:
    """One `.safetensors` file, memory-mapped: `names()` and `tensor(name)` (a copy; the map is closed with the object)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
        (n,) = struct.unpack("<Q", head)
        size = os.fstat(self._f.fileno()).st_size
        if n < 2 or 8 + n > size:
            raise ValueError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        self._entries = json.loads(self._f.read(n).decode("utf-8"))
        self._entries.pop("__metadata__", None)
        self._base = 8 + n
        end = max((e["data_offsets"][1] for e in self._entries.values()), default=0)
        if self._base + end > size:
            raise ValueError(f"{path}: the header claims {end} data bytes, the file holds {size - self._base}")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self) -> list[str]:
        return list(self._entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self._entries[name]
        if e["dtype"] not in _DTYPES:
            raise ValueError(f"{self.path}: {name} has dtype {e['dtype']}, which this loader does not read")
        dt, shape = _DTYPES[e["dtype"]], tuple(e["shape"])
        a, b = e["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if b - a != count * dt.itemsize or self._base + b > len(self._map):
            raise ValueError(f"{self.path}: {name} claims {b - a} bytes at {a} for shape {shape} {e['dtype']}")
        if count == 0:
            return torch.empty(shape, dtype=dt)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=b - a, offset=self._base + a).copy()
        return torch.from_numpy(raw).view(dt).reshape(shape)

    def close(self) -> None:
        self._map.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def read_config(path: str) -> DecoderConfig:
    """The decoder fields of `config.json` (transformers' CohereAsrConfig as written by save_pretrained)."""
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    enc = c.get("encoder_config") or {}
    return DecoderConfig(
        vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], num_hidden_layers=c["num_hidden_layers"],
        num_attention_heads=heads, num_key_value_heads=c.get("num_key_value_heads", heads),
        head_dim=c.get("head_dim", c["hidden_size"] // heads), intermediate_size=c["intermediate_size"],
        hidden_act=c.get("hidden_act", "relu"), max_position_embeddings=c["max_position_embeddings"],
        pad_token_id=c.get("pad_token_id", 2), eos_token_id=c.get("eos_token_id", 3),
        bos_token_id=c.get("bos_token_id", 4), encoder_hidden_size=enc.get("hidden_size", c["hidden_size"]),
        layer_norm_eps=c.get("layer_norm_eps", 1e-5),
        extra={"subsampling_factor": enc.get("subsampling_factor", 8)})


def _files(path: str) -> list[str]:
    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index):  # sharded: only the shards that hold a decoder tensor
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        return sorted({os.path.join(path, fn) for name, fn in weight_map.items() if module_name(name)})
    single = os.path.join(path, "model.safetensors")
    if os.path.exists(single):
        return [single]
    found = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
    if not found:
        raise FileNotFoundError(f"{path}: no model.safetensors, no index, no *.safetensors")
    return found


def load_decoder(path: str, dtype: torch.dtype | None = None) -> SyntheticCohereAsr:
    """The decoder of the checkpoint directory `path` on the CPU, as a module with the attribute tree StreamDecoder
    reads. dtype: convert floating-point tensors (None: as stored; the reference loads bf16, server.py:266). Raises if a
    tensor the decoder needs is missing, has another shape, or if a decoder tensor of the file has no place."""
    cfg = read_config(path)
    if cfg.extra["subsampling_factor"] != 8:
        raise ValueError(f"{path}: encoder subsampling factor {cfg.extra['subsampling_factor']}, expected 8")
    model = SyntheticCohereAsr(cfg)
    want = dict(model.state_dict())
    got: dict[str, torch.Tensor] = {}
    for fn in _files(path):
        with SafetensorsFile(fn) as sf:
            for name in sf.names():
                key = module_name(name)
                if key is None:
                    continue
                if key not in want:
                    raise KeyError(f"{fn}: decoder tensor {name} (-> {key}) has no place in the decoder")
                t = sf.tensor(name)
                if tuple(t.shape) != tuple(want[key].shape):
                    raise ValueError(f"{fn}: {name} has shape {tuple(t.shape)}, the config gives {tuple(want[key].shape)}")
                got[key] = t
    missing = sorted(set(want) - set(got))
    if missing:
        raise KeyError(f"{path}: {len(missing)} decoder tensors missing, e.g. {missing[:4]}")
    for key, t in got.items():  # parameters are replaced, not copied into: the stored dtype survives
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        mod = model
        *parents, leaf = key.split(".")
        for p in parents:
            mod = getattr(mod, p)
        setattr(mod, leaf, torch.nn.Parameter(t, requires_grad=False))
    return model.eval()
