"""oracle/decoder.py against transformers' CohereAsrDecoder + proj_out (the reference's FAST=0 arithmetic), through the
vectors of tests/golden/decoder_*.npz."""

import os

import numpy as np
import pytest

from cohere_inference_b200.synth import config1_inputs, synthetic_model
from oracle.decoder import (OracleConfig, OracleDecoder, StreamOracle, argmax_first, effective_weights,
                            state_to_numpy)


@pytest.mark.parametrize("tag,heads,hd,act,bias", [("gelu", 4, 16, "gelu", 0.05), ("relu", 2, 32, "relu", 0.0)])
def test_small_model_logits(golden_dir, tag, heads, hd, act, bias):
    g = np.load(os.path.join(golden_dir, "decoder_small.npz"))
    model = synthetic_model(1, heads=heads, head_dim=hd, act=act, layers=2, hidden=64, ffn=128, vocab=96, max_pos=32,
                            bias_std=bias)
    w = effective_weights(state_to_numpy(model), 2)
    dec = OracleDecoder(w, OracleConfig.of(model.config))
    memory, lens, tokens, want = (g[f"{tag}_{k}"] for k in ("memory", "lens", "tokens", "logits"))
    cross = [dec.cross_kv(memory[r, :lens[r]]) for r in range(3)]
    caches = [dec.new_self_cache() for _ in range(3)]
    for t in range(tokens.shape[1]):  # a ragged batch in one call
        logits = dec.step(tokens[:, t], np.full(3, t), caches, cross)
        np.testing.assert_allclose(logits, want[:, t], atol=2e-5, rtol=1e-5)


def test_config1_greedy_matches_transformers(golden_dir):
    """BASELINE config 1: batch 1, fp32, 8 layers x 1024, 16 heads x 64, GELU, vocab 16384, 125 frames, 10 + 64 tokens."""
    g = np.load(os.path.join(golden_dir, "decoder_config1.npz"))
    model = synthetic_model(0)
    memory, prompt = config1_inputs(0)
    assert abs(float(memory.astype(np.float64).sum()) - float(g["memory_checksum"])) < 1e-6
    assert np.array_equal(prompt, g["prompt"])
    w = effective_weights(state_to_numpy(model), 8)
    so = StreamOracle(w, OracleConfig.of(model.config), slots=1, max_new_tokens=64, max_prompt=16, eos=-1, record=True)
    so.fill_cross(memory[0], [125], [0])
    so.admit([0], [prompt[0]], [125])
    b = so.set_active([0])
    for _ in range(73):
        so.step(b)
    assert so.finished[0] == 1 and so.pos[0] == 73
    fed = np.array([r[2] for r in so.record])
    assert np.array_equal(fed, np.arange(73))
    logits = np.stack([r[3] for r in so.record])
    np.testing.assert_allclose(logits[:, ::64], g["logits_sub"], atol=1e-4, rtol=0)
    assert np.array_equal(argmax_first(logits), g["argmax"])
    assert np.array_equal(so.out[0, :10], prompt[0]) and np.array_equal(so.out[0, 10:74], g["argmax"][9:])


@pytest.mark.parametrize("name,rows", [("config2", (0,)), ("config3", (0, 63)), ("config3_kv8", (5,)), ("sparse128", (127,))])
def test_full_size_goldens_pin_the_oracle(golden_dir, name, rows):
    """The full-size goldens (transformers on the weights each mode stores) against the numpy oracle on a few rows:
    teacher-forced along the golden's own tokens, the first 13 steps, logits at every 256th entry and the top logit."""
    from cohere_inference_b200.synth import parity_workload
    g = np.load(os.path.join(golden_dir, f"decoder_{name}.npz"))
    wl = parity_workload(name)
    assert np.array_equal(g["frames"], wl.frames)
    assert abs(sum(float(m.astype(np.float64).sum()) for m in wl.memory) - float(g["memory_checksum"])) < 1e-6
    assert np.array_equal(g["seq"][:, :wl.prompts.shape[1]], wl.prompts)
    model = synthetic_model(0)
    w = effective_weights(state_to_numpy(model), 8, wl.mode, tables="bf16")
    dec = OracleDecoder(w, OracleConfig.of(model.config), kv_round="int8" if wl.kv_int8 else None)
    # int8 caches: a last-bit difference between the two fp32 computations can move a cached value by one quantisation
    # step (scale = absmax / 127), which shows in the logits at the 1e-4 level
    tol = 1e-3 if wl.kv_int8 else 1e-4
    for r in rows:
        cross, cache = [dec.cross_kv(wl.memory[r])], [dec.new_self_cache()]
        for t in range(13):
            assert g["fed"][r, t] == g["seq"][r, t]
            logits = dec.step(g["fed"][r, t:t + 1].astype(np.int64), np.array([t]), cache, cross)[0]
            assert abs(float(logits[g["argmax"][r, t]]) - float(g["top1"][r, t])) <= tol
            if g["gap"][r, t] > 10 * tol:
                assert int(argmax_first(logits)) == int(g["argmax"][r, t])
            if t % 4 == 0:
                np.testing.assert_allclose(logits[::256], g["logits_sub"][r, t // 4], atol=tol, rtol=0)
