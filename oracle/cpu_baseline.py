"""TEST INFRASTRUCTURE, not product code: the CPU arithmetic of the path, timed on the host cores.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this package.

Two arms, same weights (the seed's synthetic model) and the same shapes as the GPU workload:
  "reference"  the reference's FAST=0 arithmetic: transformers' CohereAsrDecoder + proj_out in fp32 with its KV cache,
               driven by a manual greedy loop (server.py:263-267, 311-324 of the reference load and call this model;
               transformers/models/cohere_asr/modeling_cohere_asr.py holds the arithmetic). Used when transformers
               imports on the box.
  "port"       oracle/decoder.py (numpy), the restatement pinned against it.
Both decode a bounded sample: `steps` decoding steps of a batch of `batch` rows from position 0 with ragged encoder
lengths, after computing the cross keys/values once (the prefill is timed separately and not counted in tokens/s).
A step's CPU cost is dominated by the projections (2 * 134 M MACs per row), not by the position, so early positions
stand for the whole sequence.
"""

from __future__ import annotations

import os
import time

import numpy as np
import torch


def hf_model(synth):
    """The transformers model class the reference serves, loaded with the synthetic model's weights."""
    from transformers.models.cohere_asr import modeling_cohere_asr as m
    from transformers.models.cohere_asr.configuration_cohere_asr import CohereAsrConfig
    c = synth.config
    cfg = CohereAsrConfig(vocab_size=c.vocab_size, hidden_size=c.hidden_size, num_hidden_layers=c.num_hidden_layers,
                          num_attention_heads=c.num_attention_heads, num_key_value_heads=c.num_key_value_heads,
                          head_dim=c.head_dim, intermediate_size=c.intermediate_size, hidden_act=c.hidden_act,
                          max_position_embeddings=c.max_position_embeddings,
                          encoder_config=dict(hidden_size=c.encoder_hidden_size, num_hidden_layers=1))
    model = m.CohereAsrForConditionalGeneration(cfg).eval()
    missing, unexpected = model.load_state_dict(synth.state_dict(), strict=False)
    assert not unexpected and all(k.startswith("model.encoder") for k in missing), (missing[:5], unexpected[:5])
    return model


def _inputs(batch: int, seed: int, frames=(50, 375), prompt_len: int = 10, vocab: int = 16384, hidden: int = 1024):
    rng = np.random.default_rng(seed)
    lens = rng.integers(frames[0], frames[1] + 1, batch)
    memory = [rng.standard_normal((int(t), hidden), dtype=np.float32) for t in lens]
    prompts = rng.integers(0, vocab, (batch, prompt_len)).astype(np.int64)
    return lens, memory, prompts


@torch.no_grad()
def time_reference(synth, batch: int, steps: int, seed: int = 0) -> dict:
    """transformers on the host cores: padded batch with an encoder attention mask, greedy, prompt forced."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    model = hf_model(synth)
    lens, memory, prompts = _inputs(batch, seed, vocab=synth.config.vocab_size, hidden=synth.config.hidden_size)
    T = int(max(lens))
    mem = torch.zeros(batch, T, synth.config.hidden_size)
    mask = torch.zeros(batch, T, dtype=torch.long)
    for r, m in enumerate(memory):
        mem[r, :len(m)] = torch.from_numpy(m)
        mask[r, :len(m)] = 1
    dec, past = model.model.decoder, None
    tok = torch.from_numpy(prompts[:, :1])
    t0 = time.perf_counter()
    o = dec(input_ids=tok, encoder_hidden_states=mem, encoder_attention_mask=mask, past_key_values=past, use_cache=True)
    past = o.past_key_values
    nxt = model.proj_out(o.last_hidden_state[:, -1]).argmax(-1)
    t_first = time.perf_counter() - t0  # includes the cross K/V of all layers (the prefill)
    t0 = time.perf_counter()
    for t in range(1, steps + 1):
        tok = torch.from_numpy(prompts[:, t:t + 1]) if t < prompts.shape[1] else nxt[:, None]
        o = dec(input_ids=tok, encoder_hidden_states=mem, encoder_attention_mask=mask, past_key_values=past,
                use_cache=True)
        past = o.past_key_values
        nxt = model.proj_out(o.last_hidden_state[:, -1]).argmax(-1)
    dt = time.perf_counter() - t0
    return dict(kind="reference", cores=threads, seconds=dt, steps=steps, batch=batch, tokens_per_s=batch * steps / dt,
                ms_per_step=1e3 * dt / steps, prefill_s=t_first,
                sample=f"transformers {_tf_version()} CohereAsrDecoder fp32, batch {batch}, {steps} cached greedy steps "
                       f"from position 1, encoder lengths U[50,375]; first step with cross-K/V prefill "
                       f"{t_first:.1f} s not counted")


def _tf_version() -> str:
    try:
        import transformers
        return transformers.__version__
    except Exception:  # pragma: no cover
        return "?"


def time_port(synth, batch: int, steps: int, seed: int = 0) -> dict:
    """oracle/decoder.py (numpy) on the host cores."""
    from .decoder import OracleConfig, OracleDecoder, argmax_first, effective_weights, state_to_numpy
    threads = os.cpu_count() or 1
    w = effective_weights(state_to_numpy(synth), synth.config.num_hidden_layers)
    dec = OracleDecoder(w, OracleConfig.of(synth.config))
    lens, memory, prompts = _inputs(batch, seed, vocab=synth.config.vocab_size, hidden=synth.config.hidden_size)
    t0 = time.perf_counter()
    cross = [dec.cross_kv(m) for m in memory]
    t_prefill = time.perf_counter() - t0
    caches = [dec.new_self_cache() for _ in range(batch)]
    tok = prompts[:, 0]
    logits = dec.step(tok, np.zeros(batch, np.int64), caches, cross)
    t0 = time.perf_counter()
    for t in range(1, steps + 1):
        tok = prompts[:, t] if t < prompts.shape[1] else argmax_first(logits)
        logits = dec.step(tok, np.full(batch, t), caches, cross)
    dt = time.perf_counter() - t0
    return dict(kind="port", cores=threads, seconds=dt, steps=steps, batch=batch, tokens_per_s=batch * steps / dt,
                ms_per_step=1e3 * dt / steps, prefill_s=t_prefill,
                sample=f"numpy port of the decoder (oracle/decoder.py), batch {batch}, {steps} cached greedy steps from "
                       f"position 1, encoder lengths U[50,375]; cross-K/V prefill {t_prefill:.1f} s not counted")


def time_cpu(synth, batch: int, steps: int, seed: int = 0, prefer: str = "reference") -> dict:
    if prefer == "reference":
        try:
            return time_reference(synth, batch, steps, seed)
        except Exception as e:  # transformers missing or incompatible on this box: fall back to the port
            out = time_port(synth, batch, steps, seed)
            out["sample"] += f" (transformers arm unavailable: {type(e).__name__}: {e})"[:200]
            return out
    return time_port(synth, batch, steps, seed)
