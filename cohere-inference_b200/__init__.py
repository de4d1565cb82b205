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
    import importlib
    if name == "StreamDecoder":
        return importlib.import_module(__name__ + ".stream_decoder").StreamDecoder
    if name == "DecodeScheduler":
        return importlib.import_module(__name__ + ".scheduler").DecodeScheduler
    if name in ("native", "packing", "scheduler", "stream_decoder", "synth", "build"):
        return importlib.import_module(__name__ + "." + name)
    raise AttributeError(name)
