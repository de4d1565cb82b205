"""The drop-in under the reference's own Pipeline (kernels/pipeline.py: encoder thread, `_take`, the fill_cross
hand-off, the decoder thread with its one-step-behind flag reads). Optional: it needs a checkout of the reference,
named by the environment variable B200DEC_REFERENCE_ROOT, and is skipped without one. The reference's encoder and
feature extractor (out of scope here, and in need of the gated checkpoint) are replaced by stubs that turn a piece of
"audio" into seeded N(0, 1) encoder frames; `kernels.stream_decoder.StreamDecoder` is this package's class. Every
request's tokens are compared with the CPU oracle decoding it alone."""

import os
import sys
import types

import numpy as np
import pytest
import torch

from cohere_inference_b200.synth import synthetic_model
from oracle.decoder import OracleConfig, StreamOracle, effective_weights, state_to_numpy

REF = os.environ.get("B200DEC_REFERENCE_ROOT", "")
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(os.path.join(REF, "kernels", "pipeline.py")),
                                 reason="set B200DEC_REFERENCE_ROOT to a checkout of the reference to run this")]


def _memory(seed: int, frames: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((frames, 1024), dtype=np.float32)


def _install_stubs(decoder_cls):
    """Stand-ins for the modules kernels/pipeline.py imports at its top."""
    feats = types.ModuleType("kernels.features")

    class Features:  # log-mel features: here the pieces pass through
        def __init__(self, extractor):
            pass

        def __call__(self, pieces):
            return pieces, [int(p.numel()) // 1280 + 1 for p in pieces]
    feats.Features, feats.dither = Features, (lambda x: x)
    enc = types.ModuleType("kernels.fast_encoder")

    class FastEncoder:  # a piece's first sample carries its seed; its length decides its frames (as _take counts them)
        def __init__(self, encoder, int8=False, sparse=None):
            pass

        def __call__(self, pieces, frames):
            rows = [torch.from_numpy(_memory(int(p[0].item()), f)) for p, f in zip(pieces, frames)]
            return torch.cat(rows).to(pieces[0].device).to(torch.bfloat16), list(frames)
    enc.FastEncoder = FastEncoder
    dec = types.ModuleType("kernels.stream_decoder")
    dec.StreamDecoder = decoder_cls
    pkg = types.ModuleType("kernels")
    pkg.__path__ = [os.path.join(REF, "kernels")]
    for name, mod in (("kernels", pkg), ("kernels.features", feats), ("kernels.fast_encoder", enc),
                      ("kernels.stream_decoder", dec)):
        sys.modules[name] = mod


def test_reference_pipeline_drives_this_decoder():
    from cohere_inference_b200 import StreamDecoder
    _install_stubs(StreamDecoder)
    import importlib
    Pipeline = importlib.import_module("kernels.pipeline").Pipeline
    model = synthetic_model(0, layers=2)
    pipe = Pipeline(model.cuda(), None, slots=4, max_new_tokens=24, int8=True)
    assert type(pipe.decoder) is StreamDecoder
    rng = np.random.default_rng(9)
    jobs = []
    for j in range(6):  # 6 requests of 1-3 pieces each through 4 slots
        pieces = []
        for _ in range(int(rng.integers(1, 4))):
            frames = int(rng.integers(20, 120))
            x = np.zeros((frames - 1) * 1280 + 7, np.float32)
            x[0] = float(rng.integers(1, 1 << 20))  # the stub encoder's seed
            pieces.append(x)
        prompt = torch.from_numpy(rng.integers(4, 16384, int(rng.integers(2, 9))).astype(np.int64))
        limits = [int(rng.integers(3, 24)) for _ in pieces]
        jobs.append((pieces, prompt, limits, pipe.submit(pieces, prompt, limits)))
    w = effective_weights(state_to_numpy(model), 2, "int8", tables="bf16")
    same = total = 0
    for pieces, prompt, limits, fut in jobs:
        got = fut.result(timeout=120)
        assert len(got) == len(pieces)
        for x, limit, row in zip(pieces, limits, got):
            frames = len(x) // 1280 + 1
            so = StreamOracle(w, OracleConfig.of(model.config), slots=1, max_new_tokens=24, max_prompt=16,
                              frames=pipe.decoder.frames)
            # the stub hands the frames over as bf16, as the reference's encoder does
            mem = torch.from_numpy(_memory(int(x[0]), frames)).to(torch.bfloat16).float().numpy()
            so.fill_cross(mem, [frames], [0])
            so.admit([0], [prompt.numpy()], [frames], [limit])
            b = so.set_active([0])
            while not so.finished[0]:
                so.step(b)
            n = int(so.pos[0]) + 1
            want = so.out[0, :n]
            assert np.array_equal(row[:len(prompt)], prompt.numpy())
            diff = np.nonzero(row[:min(len(row), n)] != want[:min(len(row), n)])[0]
            k = diff[0] if len(diff) else min(len(row), n)
            same += k - len(prompt)
            total += (k - len(prompt)) + (1 if len(diff) else 0)
            if not len(diff):  # the reference delivers up to max_new_tokens: past a piece's own limit only padding
                assert len(row) >= n and (row[n:] == pipe.decoder.pad).all()
    pipe.decoder.check_status()
    print(f"reference Pipeline over this decoder: {same}/{total} generated tokens equal to the oracle before the first "
          f"divergence, {pipe.stats['steps']} steps, {pipe.stats['chunks']} encoder chunks")
    assert total > 0 and same / total >= 0.97
