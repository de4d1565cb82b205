"""Seeded random-init decoder with the attribute tree of transformers' CohereAsrForConditionalGeneration.

StreamDecoder (like the reference's, kernels/stream_decoder.py:51-62, 73-99) reads a model only through
`model.config`, `model.model.decoder.*`, `model.proj_out` and `model.model.encoder._get_subsampling_output_length`.
This module builds that tree from plain torch.nn modules without transformers, so benchmarks and tests do not need a
checkpoint: Linear and Embedding weights N(0, 0.02), LayerNorm weight 1 / bias 0, Linear biases 0 (what
transformers' `_init_weights` gives, transformers/models/cohere_asr/modeling_cohere_asr.py:323-345), the pad row of the
token embedding zero, and `decoder.proj` the identity so a [B, T, d_model] memory passes through unchanged.

The numbers come from numpy's PCG64 stream (platform-independent), drawn parameter by parameter in
module registration order, so the same seed gives bit-identical fp32 weights on every machine. `state_dict()` keys equal the
transformers ones, so the same weights load into the real CohereAsr model (tests/golden/make_golden.py does that).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace

import numpy as np
import torch
from torch import nn


@dataclass
class DecoderConfig:
    """The fields of transformers' CohereAsrConfig that the decoder path reads."""
    vocab_size: int = 16384
    hidden_size: int = 1024
    num_hidden_layers: int = 8
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    head_dim: int = 64
    intermediate_size: int = 4096
    hidden_act: str = "gelu"
    max_position_embeddings: int = 1024
    pad_token_id: int = 2
    eos_token_id: int = 3
    bos_token_id: int = 4
    encoder_hidden_size: int = 1024
    layer_norm_eps: float = 1e-5
    extra: dict = field(default_factory=dict)


class _Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        d, hd = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(d, hd), nn.Linear(d, hd), nn.Linear(d, hd)
        self.o_proj = nn.Linear(hd, d)


class _MLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.fc1 = nn.Linear(cfg.hidden_size, cfg.intermediate_size)
        self.fc2 = nn.Linear(cfg.intermediate_size, cfg.hidden_size)


class _Layer(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.self_attn, self.encoder_attn, self.mlp = _Attention(cfg), _Attention(cfg), _MLP(cfg)
        eps = cfg.layer_norm_eps
        self.input_layernorm = nn.LayerNorm(cfg.hidden_size, eps=eps)
        self.post_attention_layernorm = nn.LayerNorm(cfg.hidden_size, eps=eps)
        self.final_layernorm = nn.LayerNorm(cfg.hidden_size, eps=eps)


class _Decoder(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([_Layer(cfg) for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.pos_emb = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size)
        self.embedding_layernorm = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_eps)
        self.proj = nn.Linear(cfg.encoder_hidden_size, cfg.hidden_size)


class _EncoderStub(nn.Module):
    """Only the frame-count rule of the real encoder: 8x subsampling by three stride-2 convolutions
    (1001 feature frames -> 126, 3001 -> 376, 3601 -> 451)."""

    @staticmethod
    def _get_subsampling_output_length(n: torch.Tensor) -> torch.Tensor:
        for _ in range(3):
            n = torch.div(n - 1, 2, rounding_mode="floor") + 1
        return n


class _Inner(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.decoder = _Decoder(cfg)
        self.encoder = _EncoderStub()


class SyntheticCohereAsr(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.config = cfg
        self.model = _Inner(cfg)
        self.proj_out = nn.Linear(cfg.hidden_size, cfg.vocab_size)


def synthetic_model(seed: int = 0, *, heads: int = 16, head_dim: int = 64, act: str = "gelu", layers: int = 8,
                    hidden: int = 1024, ffn: int = 4096, vocab: int = 16384, max_pos: int = 1024,
                    bias_std: float = 0.0, dtype: torch.dtype = torch.float32) -> SyntheticCohereAsr:
    """The seed's model. bias_std > 0 also draws every Linear bias and LayerNorm bias from N(0, bias_std) and the
    LayerNorm weights from 1 + N(0, bias_std): the init of transformers leaves those at 0 / 1, which would leave the
    bias and affine code paths untested."""
    cfg = DecoderConfig(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                        num_key_value_heads=heads, head_dim=head_dim, intermediate_size=ffn, hidden_act=act,
                        max_position_embeddings=max_pos, encoder_hidden_size=hidden)
    model = SyntheticCohereAsr(cfg)
    rng = np.random.default_rng(seed)

    def normal(shape, std, mean=0.0):
        return torch.from_numpy((rng.standard_normal(shape, dtype=np.float32) * np.float32(std)
                                 + np.float32(mean)).astype(np.float32))

    with torch.no_grad():
        for name, p in model.named_parameters():  # registration order
            if name.endswith("decoder.proj.weight"):
                p.copy_(torch.eye(p.shape[0], p.shape[1]))
            elif name.endswith("decoder.proj.bias"):
                p.zero_()
            elif p.dim() == 2:
                p.copy_(normal(p.shape, 0.02))
            elif "layernorm" in name or name.endswith("decoder.norm.weight") or name.endswith("decoder.norm.bias"):
                if name.endswith("weight"):
                    p.copy_(normal(p.shape, bias_std, 1.0) if bias_std else torch.ones_like(p))
                else:
                    p.copy_(normal(p.shape, bias_std) if bias_std else torch.zeros_like(p))
            else:  # Linear bias
                p.copy_(normal(p.shape, bias_std) if bias_std else torch.zeros_like(p))
        model.model.decoder.embed_tokens.weight[cfg.pad_token_id].zero_()
    return model.to(dtype).eval()


def synthetic_requests(n: int, seed: int = 0, *, vocab: int = 16384, prompt_len: int = 10, frames=(50, 375),
                       targets=(16, 448), slots: int = 128, fill: float = 0.95) -> list[SimpleNamespace]:
    """A seeded stream of n decode requests: encoder frames uniform in frames, tokens to generate uniform in targets,
    a prompt of prompt_len uniform token ids, Poisson arrivals in units of decoding steps at the rate that keeps
    `slots` slots `fill` full (rate = fill * slots / mean steps per request, a request taking prompt_len - 1 + target
    steps). Each item: .frames .target .prompt (int64 array) .arrival (float, in steps) .mem_seed."""
    rng = np.random.default_rng(seed)
    t = rng.integers(frames[0], frames[1] + 1, n)
    g = rng.integers(targets[0], targets[1] + 1, n)
    prompts = rng.integers(0, vocab, (n, prompt_len))
    mean_steps = prompt_len - 1 + (targets[0] + targets[1]) / 2
    gaps = rng.exponential(mean_steps / (fill * slots), n)
    arrival = np.cumsum(gaps)
    return [SimpleNamespace(frames=int(t[i]), target=int(g[i]), prompt=prompts[i].astype(np.int64),
                            arrival=float(arrival[i]), mem_seed=int(seed * 1_000_003 + i)) for i in range(n)]


def config1_inputs(seed: int = 0, batch: int = 1, frames: int = 125, prompt_len: int = 10, hidden: int = 1024,
                   vocab: int = 16384) -> tuple[np.ndarray, np.ndarray]:
    """Encoder memory (batch, frames, hidden) ~ N(0, 1) fp32 and prompts (batch, prompt_len) uniform over the
    vocabulary, from numpy's PCG64 stream of the seed (the same numbers on every machine)."""
    rng = np.random.default_rng(seed)
    memory = rng.standard_normal((batch, frames, hidden), dtype=np.float32)
    prompt = rng.integers(0, vocab, (batch, prompt_len)).astype(np.int64)
    return memory, prompt


# The benchmark configurations as parity workloads: the golden generator (tests/golden/make_golden.py, transformers on
# the CPU) and the GPU tests build their inputs from here, so both sides see the same numbers.
PARITY_WORKLOADS = {
    # name: (rows, frames (lo, hi), prompt tokens, new tokens, weight mode, int8 KV caches, input seed)
    "config2": (8, (375, 375), 10, 448, "bf16", False, 1002),
    "config3": (64, (50, 375), 10, 448, "int8", False, 1000),
    "config3_kv8": (64, (50, 375), 10, 448, "int8", True, 1000),
    "sparse128": (128, (50, 375), 10, 64, "int8_24", False, 1004),
}


def parity_workload(name: str, hidden: int = 1024, vocab: int = 16384) -> SimpleNamespace:
    """Inputs of one benchmark configuration at full size: .rows, .frames (list), .memory (list of (frames, hidden)
    fp32 arrays ~ N(0, 1)), .prompts (rows, plen) int64, .new, .mode (weight storage: bf16 / int8 / int8_24),
    .kv_int8; all from numpy's PCG64 stream of the workload's seed."""
    rows, (lo, hi), plen, new, mode, kv8, seed = PARITY_WORKLOADS[name]
    rng = np.random.default_rng(seed)
    frames = rng.integers(lo, hi + 1, rows).tolist()
    memory = [rng.standard_normal((t, hidden), dtype=np.float32) for t in frames]
    prompts = rng.integers(0, vocab, (rows, plen)).astype(np.int64)
    return SimpleNamespace(name=name, rows=rows, frames=frames, memory=memory, prompts=prompts, new=new, mode=mode,
                           kv_int8=kv8)


def request_memory(req, hidden: int = 1024) -> np.ndarray:
    """Encoder memory (frames, hidden) ~ N(0, 1) fp32 of a synthetic request, from its own seed."""
    return np.random.default_rng(req.mem_seed).standard_normal((req.frames, hidden), dtype=np.float32)
