"""Generates the golden vectors in this directory. Run once in the build container, where the reference checkout and
transformers are present; the tests only read the .npz files.

    python tests/golden/make_golden.py /path/to/reference

packers.npz   outputs of the reference's own pure-torch packers (kernels/stream_decoder.py prepare_w8,
              kernels/fast_encoder.py quantize_rows maths, kernels/sparse.py prune_24_magnitude / compress_24) on seeded
              inputs. kernels/cuda_ext.py (the JIT build, needs a GPU) is stubbed out before import; nothing else of
              the reference runs.
decoder_small.npz  transformers' CohereAsrDecoder + proj_out (the reference's FAST=0 arithmetic) on a small seeded
              model, ragged batch, full logits per step.
decoder_config1.npz  the same model class at the benchmark architecture (8 layers, 1024 wide, 16 heads x 64, GELU, vocab
              16384), batch 1, memory [1, 125, 1024], 10-token prompt + 64 forced new tokens, seed 0, fp32: greedy
              argmax of all 73 steps and the logits at every 64th vocabulary entry.
decoder_config2.npz, decoder_config3.npz, decoder_config3_kv8.npz, decoder_sparse128.npz
              the benchmark configurations at full size (cohere_inference_b200.synth.PARITY_WORKLOADS): the same
              transformers model loaded with the weights the mode stores (bf16-rounded / int8-dequantised / 2:4-pruned
              and dequantised, oracle.decoder.effective_weights), a padded batch with an encoder attention mask, greedy
              with the prompt forced. Per row and step: the token fed, the un-forced argmax, the top logit, the gap to
              the runner-up, and (every 4th step) the logits at every 256th vocabulary entry. The kv8 file keeps keys
              and values the way an int8 cache does (a Cache subclass rounds them on entry, see RoundingCache).
stream300.npz the first 300 requests of synthetic_requests(seed 0), each decoded greedily on its own (as one padded
              batch) with the 2:4 model: the token sequence every request must deliver through the scheduler.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import cohere_inference_b200 as cib  # noqa: E402
from cohere_inference_b200.synth import config1_inputs, synthetic_model  # noqa: E402


def reference_packers(ref: str):
    sys.path.insert(0, ref)
    stub = types.ModuleType("kernels.cuda_ext")
    stub.ext = None
    sys.modules["kernels.cuda_ext"] = stub
    tri = types.ModuleType("kernels.decoder_kernels")  # Triton kernels: not needed by the packers
    tri.linear = None
    sys.modules["kernels.decoder_kernels"] = tri
    from kernels.sparse import compress_24, prune_24_magnitude
    from kernels.stream_decoder import prepare_w8
    return prepare_w8, prune_24_magnitude, compress_24


def make_packers(ref: str) -> None:
    prepare_w8, prune_24_magnitude, compress_24 = reference_packers(ref)
    rng = np.random.default_rng(0)
    out = {}
    cases = {"a": (48, 64), "b": (16, 256), "c": (32, 1024)}
    for name, (n, k) in cases.items():
        w = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
        if name == "a":
            w[3] = 0  # an all-zero row: scale clamps at 1e-12 / 127
            w[5, :8] = [0.5, -0.5, 0.25, 0.25, 0, 0, 0, 1e-3]  # ties and zeros inside groups of four
            w[7] *= 1e-9
        t = torch.from_numpy(w)
        u8, s = prepare_w8(t)
        pruned = prune_24_magnitude(t)
        sp = pruned.float().abs().amax(1).clamp_min(1e-12) / 127  # quantize_rows' maths (fast_encoder.py:60-63)
        qp = torch.round(pruned.float() / sp[:, None]).clamp(-127, 127).to(torch.int8)
        kept, words = compress_24(qp)
        out.update({f"{name}_w": w, f"{name}_u8": u8.numpy(), f"{name}_s": s.numpy(), f"{name}_pruned": pruned.numpy(),
                    f"{name}_qp": qp.numpy(), f"{name}_sp": sp.numpy(), f"{name}_kept": kept.numpy(),
                    f"{name}_words": words.numpy()})
    # a hand-made int8 matrix with 0, 1 and 2 nonzeros per group in every position pattern
    pat = []
    for i0 in range(4):
        for i1 in range(i0 + 1, 4):
            g = [0, 0, 0, 0]
            g[i0], g[i1] = 5 + i0, -(7 + i1)
            pat.append(g)
    for i0 in range(4):
        g = [0, 0, 0, 0]
        g[i0] = -3 - i0
        pat.append(g)
    pat.append([0, 0, 0, 0])
    pat += pat[:5]
    q = np.array(pat, dtype=np.int8).reshape(2, 32)
    kept, words = compress_24(torch.from_numpy(q))
    out.update({"p_q": q, "p_kept": kept.numpy(), "p_words": words.numpy()})
    np.savez_compressed(os.path.join(HERE, "packers.npz"), **out)


def hf_model(synth):
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


@torch.no_grad()
def hf_teacher_forced(model, memory: torch.Tensor, tokens: torch.Tensor) -> np.ndarray:
    """Logits (B, steps, V) of feeding tokens[:, t] at position t with a KV cache, one token per call: the manual loop
    over model.model.decoder + proj_out (generate() cannot take a bare encoder output for this model)."""
    dec, past, rows = model.model.decoder, None, []
    for t in range(tokens.shape[1]):
        o = dec(input_ids=tokens[:, t:t + 1], encoder_hidden_states=memory, past_key_values=past, use_cache=True)
        past = o.past_key_values
        rows.append(model.proj_out(o.last_hidden_state[:, -1]).float().numpy())
    return np.stack(rows, 1)


@torch.no_grad()
def hf_greedy(model, memory: torch.Tensor, prompt: torch.Tensor, new: int):
    """Greedy decode with the prompt forced: returns (tokens fed (steps,), logits (steps, V), argmax (steps,))."""
    dec, past = model.model.decoder, None
    tok, fed, lg, am = prompt[:, :1], [], [], []
    steps = prompt.shape[1] - 1 + new
    for t in range(steps):
        o = dec(input_ids=tok, encoder_hidden_states=memory, past_key_values=past, use_cache=True)
        past = o.past_key_values
        logits = model.proj_out(o.last_hidden_state[:, -1]).float()
        a = int(logits.argmax(-1))
        fed.append(int(tok)), lg.append(logits[0].numpy()), am.append(a)
        nxt = int(prompt[0, t + 1]) if t + 1 < prompt.shape[1] else a
        tok = torch.tensor([[nxt]])
    return np.array(fed), np.stack(lg), np.array(am)


def make_decoder_small() -> None:
    out = {}
    for tag, heads, hd, act, bias in (("gelu", 4, 16, "gelu", 0.05), ("relu", 2, 32, "relu", 0.0)):
        synth = synthetic_model(1, heads=heads, head_dim=hd, act=act, layers=2, hidden=64, ffn=128, vocab=96,
                                max_pos=32, bias_std=bias)
        model = hf_model(synth)
        g = torch.Generator().manual_seed(1)
        lens = [7, 3, 5]
        memory = torch.randn(3, 7, 64, generator=g)
        tokens = torch.randint(0, 96, (3, 6), generator=g)
        # per row on its own (no padding mask needed): ragged encoder lengths
        logits = np.stack([hf_teacher_forced(model, memory[r:r + 1, :lens[r]], tokens[r:r + 1])[0] for r in range(3)])
        out.update({f"{tag}_memory": memory.numpy(), f"{tag}_lens": np.array(lens), f"{tag}_tokens": tokens.numpy(),
                    f"{tag}_logits": logits})
    np.savez_compressed(os.path.join(HERE, "decoder_small.npz"), **out)


def make_config1() -> None:
    synth = synthetic_model(0)
    model = hf_model(synth)
    memory, prompt = (torch.from_numpy(a) for a in config1_inputs(0))
    fed, logits, am = hf_greedy(model, memory, prompt, 64)
    np.savez_compressed(os.path.join(HERE, "decoder_config1.npz"), memory_checksum=np.float64(memory.double().sum()),
                        prompt=prompt.numpy(), fed=fed, argmax=am, logits_sub=logits[:, ::64].astype(np.float32),
                        top2_gap=np.sort(logits, -1)[:, -1] - np.sort(logits, -1)[:, -2])


def effective_model(mode: str):
    """transformers' model loaded with the fp32 values the GPU mode multiplies by."""
    from oracle.decoder import effective_weights, state_to_numpy
    synth = synthetic_model(0)
    w = effective_weights(state_to_numpy(synth), synth.config.num_hidden_layers, mode, tables="bf16")
    synth.load_state_dict({k: torch.from_numpy(v) for k, v in w.items()}, strict=False)
    return hf_model(synth)


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).float()


def _q8(t: torch.Tensor) -> torch.Tensor:
    """What an int8 cache returns for vectors t (..., D): bf16-round, scale = absmax / 127 (1 for a zero vector),
    q = rint(clamp(x * (1 / scale))), x ~ q * scale; all fp32 (kernels/csrc/dec_attn.cuh:46-63 of the reference)."""
    t = _bf16(t)
    mx = t.abs().amax(-1, keepdim=True)
    sc = torch.where(mx > 0, mx / 127.0, torch.ones_like(mx))
    q = torch.round(torch.clamp(t * (1.0 / sc), -127.0, 127.0))
    return q * sc


def rounding_caches():
    """An EncoderDecoderCache whose keys and values are stored as an int8 cache would hold them. The step that appends
    a self-attention pair attends it as the bf16 values (the reference's dec_attention_q8 does, dec_attn.cuh:100-106);
    cross keys and values are read back quantised from their first use on."""
    from transformers.cache_utils import DynamicCache, EncoderDecoderCache

    class SelfQ8(DynamicCache):
        def update(self, key_states, value_states, layer_idx, *a, **kw):
            k, v = super().update(_q8(key_states), _q8(value_states), layer_idx, *a, **kw)
            k, v = k.clone(), v.clone()
            n = key_states.shape[2]
            k[:, :, -n:], v[:, :, -n:] = _bf16(key_states), _bf16(value_states)
            return k, v

    class CrossQ8(DynamicCache):
        def update(self, key_states, value_states, layer_idx, *a, **kw):
            return super().update(_q8(key_states), _q8(value_states), layer_idx, *a, **kw)

    return EncoderDecoderCache(SelfQ8(), CrossQ8())


@torch.no_grad()
def hf_batch_greedy(model, memory: list, prompts: np.ndarray, new, kv_int8: bool = False, sub_steps: int = 4,
                    sub_vocab: int = 256, log=None) -> dict:
    """Greedy decoding of a ragged batch on the CPU: memory[r] (T_r, d) zero-padded to the longest with an encoder
    attention mask, the prompt forced, `new` tokens per row (an int, or one per row: rows past their end keep
    stepping and are ignored). Returns per row and step the token fed, the un-forced argmax, the top logit and its
    gap to the runner-up, every sub_steps-th step's logits at every sub_vocab-th entry, and the sequences."""
    torch.set_num_threads(os.cpu_count() or 1)
    B, plen = prompts.shape
    new = np.full(B, new) if np.isscalar(new) else np.asarray(new)
    T, d = max(len(m) for m in memory), memory[0].shape[1]
    mem, mask = torch.zeros(B, T, d), torch.zeros(B, T, dtype=torch.long)
    for r, m in enumerate(memory):
        mem[r, :len(m)] = torch.from_numpy(m)
        mask[r, :len(m)] = 1
    steps = plen - 1 + int(new.max())
    dec, past = model.model.decoder, (rounding_caches() if kv_int8 else None)
    tok = torch.from_numpy(prompts[:, :1].copy())
    fed, am, top1, gap, sub = [], [], [], [], []
    seq = np.zeros((B, plen + int(new.max())), np.int64)
    seq[:, :plen] = prompts
    for t in range(steps):
        o = dec(input_ids=tok, encoder_hidden_states=mem, encoder_attention_mask=mask, past_key_values=past,
                use_cache=True)
        past = o.past_key_values
        logits = model.proj_out(o.last_hidden_state[:, -1]).float()
        v, i = logits.topk(2, -1)
        a = logits.argmax(-1)
        fed.append(tok[:, 0].numpy().copy()), am.append(a.numpy()), top1.append(v[:, 0].numpy())
        gap.append((v[:, 0] - v[:, 1]).numpy())
        if t % sub_steps == 0:
            sub.append(logits[:, ::sub_vocab].numpy().copy())
        nxt = torch.from_numpy(prompts[:, t + 1].copy()) if t + 1 < plen else a
        seq[:, t + 1] = nxt.numpy()
        tok = nxt[:, None]
        if log and t % 50 == 0:
            log(f"  step {t}/{steps}")
    return dict(fed=np.stack(fed, 1).astype(np.int16), argmax=np.stack(am, 1).astype(np.int16),
                top1=np.stack(top1, 1).astype(np.float32), gap=np.stack(gap, 1).astype(np.float32),
                logits_sub=np.stack(sub, 1).astype(np.float32), seq=seq.astype(np.int16), new=new.astype(np.int32))


def check_batched_equals_rows() -> None:
    """The padded, masked batch gives each row what it gets alone (small model)."""
    synth = synthetic_model(1, heads=4, head_dim=16, act="gelu", layers=2, hidden=64, ffn=128, vocab=96, max_pos=32,
                            bias_std=0.05)
    model = hf_model(synth)
    rng = np.random.default_rng(3)
    memory = [rng.standard_normal((t, 64), dtype=np.float32) for t in (7, 3, 5)]
    prompts = rng.integers(0, 96, (3, 4)).astype(np.int64)
    both = hf_batch_greedy(model, memory, prompts, 6, sub_steps=1, sub_vocab=1)
    for r in range(3):
        alone = hf_batch_greedy(model, memory[r:r + 1], prompts[r:r + 1], 6, sub_steps=1, sub_vocab=1)
        assert np.array_equal(alone["seq"][0], both["seq"][r])
        assert np.abs(alone["logits_sub"][0] - both["logits_sub"][r]).max() < 1e-5


def make_workloads(names) -> None:
    from cohere_inference_b200.synth import parity_workload
    for name in names:
        wl = parity_workload(name)
        print(name, "rows", wl.rows, "mode", wl.mode, flush=True)
        out = hf_batch_greedy(effective_model(wl.mode), wl.memory, wl.prompts, wl.new, kv_int8=wl.kv_int8,
                              log=lambda m: print(m, flush=True))
        np.savez_compressed(os.path.join(HERE, f"decoder_{name}.npz"), frames=np.array(wl.frames, np.int32),
                            memory_checksum=np.float64(sum(float(m.astype(np.float64).sum()) for m in wl.memory)),
                            **out)


def make_stream(n: int = 300) -> None:
    from cohere_inference_b200.synth import request_memory, synthetic_requests
    reqs = synthetic_requests(2000, seed=0, slots=128)[:n]
    out = hf_batch_greedy(effective_model("int8_24"), [request_memory(r) for r in reqs],
                          np.stack([r.prompt for r in reqs]), [r.target for r in reqs], sub_steps=10 ** 6,
                          log=lambda m: print(m, flush=True))
    np.savez_compressed(os.path.join(HERE, "stream300.npz"), seq=out["seq"], new=out["new"], gap=out["gap"],
                        frames=np.array([r.frames for r in reqs], np.int32))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path of the reference checkout> [part ...]")
    ref = sys.argv[1]
    only = sys.argv[2:]  # optional: the parts to (re)make
    if not only or "packers" in only:
        make_packers(ref)
    if not only or "small" in only:
        make_decoder_small()
    if not only or "config1" in only:
        make_config1()
    check_batched_equals_rows()
    from cohere_inference_b200.synth import PARITY_WORKLOADS
    make_workloads([n for n in PARITY_WORKLOADS if not only or n in only])
    if not only or "stream300" in only:
        make_stream()
    print("ok", cib.__name__)
