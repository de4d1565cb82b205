"""B200-native decoder token loop: the reference's StreamDecoder API over hand-written sm_100a CUDA kernels.

Public names: StreamDecoder (the drop-in for the reference's kernels/stream_decoder.py), DecodeScheduler (the slot
scheduler of kernels/pipeline.py's decoder thread), the weight packers, and the synthetic model / request builders.
Everything that computes goes through the C-ABI library built from csrc/ (see native.py); importing this package does
not load it, the first use does, and fails loudly when it is missing.
"""

from .synth import DecoderConfig, config1_inputs, synthetic_model, synthetic_requests  # noqa: F401

__all__ = ["DecoderConfig", "synthetic_model", "synthetic_requests", "config1_inputs", "StreamDecoder",
           "DecodeScheduler", "native"]


def __getattr__(name):
    if name == "StreamDecoder":
        from .stream_decoder import StreamDecoder
        return StreamDecoder
    if name == "DecodeScheduler":
        from .scheduler import DecodeScheduler
        return DecodeScheduler
    if name == "native":
        from . import native
        return native
    raise AttributeError(name)
