"""Writes tests/golden/checkpoint_names.json: the tensor names transformers' own `save_pretrained` gives the decoder
half of a CohereAsrForConditionalGeneration checkpoint, each with the module name (`state_dict()` key) of the tensor
that holds the same values, plus their shapes. The loader's rename table (cohere-inference_b200/checkpoint.py) is
tested against this list, so it is pinned to what transformers writes, not to a reading of its source.

Run in a container that has transformers (5.5.0 here): python tests/golden/make_checkpoint_names.py
A 2-layer model with 64-wide layers is enough: the names do not depend on the sizes.
"""

import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from cohere_inference_b200.checkpoint import SafetensorsFile  # noqa: E402


def main() -> None:
    import transformers
    from transformers.models.cohere_asr import modeling_cohere_asr as m
    from transformers.models.cohere_asr.configuration_cohere_asr import CohereAsrConfig
    torch.manual_seed(0)
    cfg = CohereAsrConfig(vocab_size=96, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=4, head_dim=16, intermediate_size=128, max_position_embeddings=32,
                          encoder_config=dict(hidden_size=80, num_hidden_layers=1, num_attention_heads=4,
                                              intermediate_size=96, subsampling_conv_channels=16))
    model = m.CohereAsrForConditionalGeneration(cfg).eval()
    with torch.no_grad():  # distinct values everywhere, so that a tensor is identified by its contents
        for i, p in enumerate(model.parameters()):
            p.copy_(torch.randn(p.shape) + i)
    state = {k: v for k, v in model.state_dict().items() if k.startswith(("model.decoder.", "proj_out."))}
    names = {}
    with tempfile.TemporaryDirectory() as d:
        model.save_pretrained(d)
        with open(os.path.join(d, "config.json")) as f:
            config = json.load(f)
        with SafetensorsFile(os.path.join(d, "model.safetensors")) as sf:
            stored = {n: sf.tensor(n) for n in sf.names()}
    for key, t in state.items():
        hits = [n for n, s in stored.items() if s.shape == t.shape and torch.equal(s, t)]
        assert len(hits) == 1, (key, hits)
        names[hits[0]] = dict(module=key, shape=list(t.shape))
    others = sorted(n for n in stored if n not in names)
    assert all(n.startswith("model.encoder.") for n in others), [n for n in others if not n.startswith("model.encoder.")]
    out = dict(transformers=transformers.__version__, decoder=names, encoder_examples=others[:12],
               config_keys=sorted(config), encoder_config_keys=sorted(config["encoder_config"]))
    with open(os.path.join(HERE, "checkpoint_names.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(len(names), "decoder tensors,", len(others), "encoder tensors")


if __name__ == "__main__":
    main()
