"""ctypes binding of libb200dec.so (include/b200dec.h): structures, prototypes, and pointer helpers for torch tensors.

The library is the only compute path: `lib()` raises if it is missing (build it with build.py or
__graft_entry__.build()); nothing here falls back to PyTorch or the CPU.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200dec.so")

W_BF16, W_INT8, W_INT8_24, W_INT8_UMMA, W_F16, W_F16_UMMA, W_INT8_24_UMMA = 0, 1, 2, 3, 4, 5, 6
A_F16, A_F32_SPLIT, A_F16_ROWS16 = 0, 1, 2
OUT_F16, OUT_F32, OUT_F32_ADD = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2
ST_TOKEN_RANGE, ST_POS_RANGE, ST_FRAMES_RANGE, ST_SLOT_RANGE, ST_TIMEOUT = 1, 2, 4, 8, 16

vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class Weight(C.Structure):
    _fields_ = [("w", vp), ("meta", vp), ("scale", vp), ("bias", vp), ("ln_g", vp), ("ln_bias", vp), ("n", i32), ("k", i32), ("kind", i32),
                ("warps", i32), ("ksplit", i32)]


class Norm(C.Structure):
    _fields_ = [("w", vp), ("b", vp), ("eps", f32), ("_pad", i32)]


class LnLink(C.Structure):
    _fields_ = [("next_gamma", vp), ("out16", vp), ("stats_out", vp), ("stats_in", vp), ("stats_slots", i32),
                ("wait_limit", i32), ("status", vp), ("withhold", i32)]


class Layer(C.Structure):
    _fields_ = [("ln1", Norm), ("ln2", Norm), ("ln3", Norm), ("qkv", Weight), ("o", Weight), ("cq", Weight),
                ("co", Weight), ("fc1", Weight), ("fc2", Weight), ("self_k", vp), ("self_v", vp), ("cross_k", vp),
                ("cross_v", vp), ("self_ks", vp), ("self_vs", vp), ("cross_ks", vp), ("cross_vs", vp)]


class Plan(C.Structure):
    _fields_ = [("layers", i32), ("heads", i32), ("head_dim", i32), ("act", i32),
                ("slots", i32), ("seq", i32), ("frames", i32), ("vocab", i32),
                ("max_prompt", i32), ("out_cols", i32), ("pad", i32), ("eos", i32),
                ("a_kind", i32), ("max_pos", i32), ("head_a_kind", i32), ("pdl", i32), ("attn_ring", i32), ("kv_int8", i32),
                ("kv_prefetch_mb", i32), ("wait_limit", i32), ("withhold", i32), ("classes", i32),
                ("embed", vp), ("pos_table", vp), ("emb_ln", Norm), ("final_ln", Norm), ("layer", C.POINTER(Layer)),
                ("head", Weight),
                ("active", vp), ("tok", vp), ("pos", vp), ("plen", vp), ("limit", vp), ("cross_len", vp),
                ("finished", vp), ("forced", vp), ("out", vp), ("flags_host", vp), ("status", vp),
                ("x", vp), ("qkv", vp), ("cq", vp), ("att", vp), ("mid", vp),
                ("attn_part", vp), ("attn_count", vp), ("head_max", vp), ("head_idx", vp),
                ("xh", vp), ("ln_stats", vp), ("sched_self", vp), ("sched_cross", vp), ("logits", vp), ("argmax", vp)]


# name -> (restype, argtypes); every symbol include/b200dec.h declares
PROTOTYPES = {
    "b200dec_last_error": (C.c_char_p, []),
    "b200dec_version": (C.c_int, []),
    "b200dec_sizeof": (C.c_int, [C.c_int]),
    "b200dec_quantize_rows": (C.c_int, [vp, C.c_int, C.c_int, vp, vp, vp]),
    "b200dec_prepare_w8": (C.c_int, [vp, C.c_int, C.c_int, vp, vp, vp]),
    "b200dec_prune24": (C.c_int, [vp, C.c_int, C.c_int, vp, vp]),
    "b200dec_compress24": (C.c_int, [vp, C.c_int, C.c_int, vp, vp, vp, vp]),
    "b200dec_tiled_bytes": (i64, [C.c_int, C.c_int, C.c_int]),
    "b200dec_tiled_meta_bytes": (i64, [C.c_int, C.c_int, C.c_int]),
    "b200dec_tile_int8": (C.c_int, [vp, C.c_int, C.c_int, vp, vp]),
    "b200dec_tile_bf16": (C.c_int, [vp, C.c_int, C.c_int, vp, vp]),
    "b200dec_tile_f16_umma": (C.c_int, [vp, C.c_int, C.c_int, vp, vp]),
    "b200dec_tile_24": (C.c_int, [vp, vp, C.c_int, C.c_int, vp, vp, vp]),
    "b200dec_tile_24_umma": (C.c_int, [vp, vp, C.c_int, C.c_int, vp, vp, vp]),
    "b200dec_embed_ln": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, Norm, Norm, vp, vp, C.c_int, C.c_int, vp,
                                   C.c_int, vp]),
    "b200dec_layer_norm": (C.c_int, [vp, Norm, vp, C.c_int, C.c_int, C.c_int, vp]),
    "b200dec_linear": (C.c_int, [C.POINTER(Weight), vp, C.c_int, C.POINTER(Norm), C.c_int, C.c_int, vp, C.c_int, C.c_int,
                                 C.c_int, C.c_int, vp]),
    "b200dec_linear_linked": (C.c_int, [C.POINTER(Weight), vp, C.c_int, C.POINTER(Norm), C.c_int, C.c_int, vp, C.c_int,
                                        C.c_int, C.c_int, C.POINTER(LnLink), C.c_int, vp]),
    "b200dec_linear_stat_slots": (C.c_int, [C.POINTER(Weight)]),
    "b200dec_ln_rows16": (C.c_int, [vp, vp, C.c_int, vp, vp, vp]),
    "b200dec_linear_fits": (C.c_int, [C.c_int] * 7),
    "b200dec_head_argmax": (C.c_int, [C.POINTER(Weight), vp, C.c_int, C.POINTER(Norm), C.c_int, C.c_int, vp, vp, vp,
                                      C.c_int, vp]),
    "b200dec_head_partials": (C.c_int, [C.POINTER(Weight)]),
    "b200dec_head_umma": (C.c_int, [C.POINTER(Weight), vp, C.POINTER(Norm), C.c_int, C.c_int, vp, vp, vp, vp, C.c_int, vp]),
    "b200dec_head_umma_linked": (C.c_int, [C.POINTER(Weight), vp, vp, C.c_int, C.POINTER(Norm), C.c_int, C.c_int, vp, vp,
                                           vp, vp, C.c_int, vp]),
    "b200dec_tile_int8_umma": (C.c_int, [vp, C.c_int, C.c_int, vp, vp]),
    "b200dec_pick": (C.c_int, [vp, vp, C.c_int, vp, C.c_int, C.c_int, vp, vp, vp, vp, C.c_int, vp, vp, vp, C.c_int,
                               C.c_int, vp, vp, C.c_int, vp]),
    "b200dec_attention": (C.c_int, [C.c_int, vp, vp, C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, f32,
                                    vp, C.c_int, C.c_int, vp, vp, vp, C.c_int, vp]),
    "b200dec_attention_scratch_floats": (i64, [C.c_int, C.c_int, C.c_int]),
    "b200dec_attention_q8": (C.c_int, [C.c_int, vp, vp, C.c_int, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int,
                                       f32, vp, C.c_int, C.c_int, vp, vp, vp, C.c_int, vp]),
    "b200dec_attention_paired_q8": (C.c_int, [C.c_int, vp, vp, C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, f32, vp,
                                              C.c_int, C.c_int, C.c_int, vp]),
    "b200dec_read_probe": (C.c_int, [vp, C.c_int, C.c_int64, vp, C.c_int, vp]),
    "b200dec_scatter_kv_q8": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                        vp]),
    "b200dec_row_schedule": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp, vp, vp]),
    "b200dec_attention_paired": (C.c_int, [C.c_int, vp, vp, C.c_int, vp, vp, C.c_int, C.c_int, C.c_int, f32, vp,
                                           C.c_int, C.c_int, C.c_int, vp]),
    "b200dec_attention_ring": (C.c_int, [C.c_int, vp, vp, C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, f32,
                                         vp, C.c_int, C.c_int, vp, vp, vp, C.c_int, vp]),
    "b200dec_attention_static": (C.c_int, [C.c_int, vp, vp, C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int,
                                           f32, vp, C.c_int, C.c_int, vp, C.c_int, vp]),
    "b200dec_scatter_kv": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "b200dec_prefill_rows_bytes": (i64, [C.c_int, C.c_int]),
    "b200dec_prefill_pack_rows": (C.c_int, [vp, C.c_int, C.c_int, C.c_int, vp, vp]),
    "b200dec_prefill_tile_weight": (C.c_int, [vp, C.c_int, C.c_int, vp, vp]),
    "b200dec_prefill_gemm": (C.c_int, [vp, C.c_int, C.c_int, vp, vp, C.c_int, C.c_int, vp, vp, C.c_int, vp, vp, vp, vp,
                                       C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp]),
    "b200dec_admit": (C.c_int, [C.POINTER(Plan), vp, C.c_int, vp, C.c_int, vp]),
    "b200dec_admit_record_ints": (C.c_int, [C.c_int]),
    "b200dec_compact_active": (C.c_int, [C.POINTER(Plan), C.c_int, vp, vp, C.c_int, vp]),
    "b200dec_step": (C.c_int, [C.POINTER(Plan), C.c_int, vp]),
    "b200dec_step_rows": (C.c_int, [C.POINTER(Plan), C.c_int, C.c_int, vp]),
    "b200dec_step_launches": (C.c_int, [C.POINTER(Plan), C.c_int]),
}

_lib = None


class NativeError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """The loaded library with prototypes set. Raises when it has not been built: there is no other compute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeError(f"{LIB_PATH} is missing: build it with `python cohere-inference_b200/build.py` "
                              "(needs nvcc); this package has no PyTorch or CPU fallback")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        for which, struct in enumerate((Weight, Norm, Layer, Plan, LnLink)):  # this binding against the built library
            if handle.b200dec_sizeof(which) != C.sizeof(struct):
                raise NativeError(f"{struct.__name__}: {C.sizeof(struct)} bytes here, {handle.b200dec_sizeof(which)} "
                                  f"in {LIB_PATH}: rebuild the library (build.py --force)")
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise NativeError(f"b200dec error {rc}: {lib().b200dec_last_error().decode()}")


def ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensors only"
    return t.data_ptr()


def stream_ptr(stream: torch.cuda.Stream | None = None) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def norm(weight: torch.Tensor, bias: torch.Tensor, eps: float) -> Norm:
    assert weight.dtype == torch.float32 and bias.dtype == torch.float32
    return Norm(ptr(weight), ptr(bias), float(eps), 0)
