"""Weight packers on the GPU with the reference's names and results, and the tiled weights the step kernels read.

prepare_w8 / quantize_rows / prune_24_magnitude / compress_24 return the same tensors as the reference functions
(kernels/stream_decoder.py:41-48, kernels/fast_encoder.py:60-63, kernels/sparse.py:26-46), bit for bit, computed by the
library's kernels. PackedLinear holds one projection re-tiled for csrc/linear.cu together with the operands the
reference-format tensors were made from, so tests can check both.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import native as nv


def _f32(w: torch.Tensor) -> torch.Tensor:
    assert w.is_cuda and w.dim() == 2
    return w.detach().float().contiguous()


def quantize_rows(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """int8 (N, K), fp32 scales (N,): s = max(absmax, 1e-12) / 127, q = clamp(round(w / s), -127, 127)."""
    w = _f32(w)
    n, k = w.shape
    q = torch.empty(n, k, dtype=torch.int8, device=w.device)
    s = torch.empty(n, dtype=torch.float32, device=w.device)
    nv.check(nv.lib().b200dec_quantize_rows(nv.ptr(w), n, k, nv.ptr(q), nv.ptr(s), nv.stream_ptr()))
    return q, s


def prepare_w8(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """The reference's dec_w8_linear operand: uint8 = int8 + 128, K reordered within every 16 (W8_PERM), fp32 scales."""
    w = _f32(w)
    n, k = w.shape
    u = torch.empty(n, k, dtype=torch.uint8, device=w.device)
    s = torch.empty(n, dtype=torch.float32, device=w.device)
    nv.check(nv.lib().b200dec_prepare_w8(nv.ptr(w), n, k, nv.ptr(u), nv.ptr(s), nv.stream_ptr()))
    return u, s


def prune_24_magnitude(w: torch.Tensor) -> torch.Tensor:
    """w with the two smallest-magnitude values of every four along K set to zero (fp32 result)."""
    w = _f32(w)
    out = torch.empty_like(w)
    nv.check(nv.lib().b200dec_prune24(nv.ptr(w), w.shape[0], w.shape[1], nv.ptr(out), nv.stream_ptr()))
    return out


def compress_24(q: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """int8 (N, K) with at most two nonzeros per four -> kept values int8 (N, K/2), selectors int32 (N, K/32)."""
    assert q.is_cuda and q.dtype == torch.int8 and q.dim() == 2 and q.shape[1] % 32 == 0
    q = q.contiguous()
    n, k = q.shape
    kept = torch.empty(n, k // 2, dtype=torch.int8, device=q.device)
    words = torch.empty(n, k // 32, dtype=torch.int32, device=q.device)
    bad = torch.zeros(1, dtype=torch.int32, device=q.device)
    nv.check(nv.lib().b200dec_compress24(nv.ptr(q), n, k, nv.ptr(kept), nv.ptr(words), nv.ptr(bad), nv.stream_ptr()))
    assert int(bad.item()) == 0, "more than two nonzero values in a group of four"
    return kept, words


# (N, K) -> (warps per CTA, CTAs per cluster along K) by weight kind: CTAs = N / (16 warps) * ksplit, K / ksplit in
# {128, 256, 512}. Chosen so every projection spreads over about one CTA per SM (148) or two.
TILE_CONFIG = {
    (3072, 1024): [(8, 4), (8, 8), (4, 8), (4, 4)],   # 96 CTAs: one wave (192 put two CTAs on 44 SMs and ran 2 us longer)
    (1024, 1024): [(4, 8), (4, 4)],
    (4096, 1024): [(8, 4), (8, 8), (4, 8), (4, 4)],   # 128 CTAs
    (1024, 4096): [(4, 8)],
    (16384, 1024): [(8, 4), (8, 8), (8, 2)],
}


def tile_config(n: int, k: int, kind: int, a_kind: int = nv.A_F16, ln: bool = False, max_rows: int = 64
                ) -> tuple[int, int]:
    """The first preferred (warps, ksplit) of the shape whose shared-memory footprint fits `max_rows` rows in one
    pass; if none does, the first valid one (the library then makes two passes of 64 rows)."""
    fits = nv.lib().b200dec_linear_fits
    prefs = TILE_CONFIG.get((n, k), []) + [(w, s) for s in (8, 4, 2, 1) for w in (4, 8)]
    kpb = {nv.W_INT8: 64, nv.W_BF16: 32, nv.W_F16: 32, nv.W_INT8_24: 128}[kind]  # k per weight block of the kind
    valid = [(w, s) for w, s in prefs if n % (16 * w) == 0 and (k, s) in ((1024, 8), (1024, 4), (1024, 2), (4096, 8))
             and (16 * w) % (8 * s) == 0 and (k // s) % kpb == 0 and (not ln or k == 1024)]
    assert valid, f"no tile for a ({n}, {k}) projection"
    for w, s in valid:
        # a LayerNorm-folding projection of an fp16-operand decoder stages the ready fp16 rows its producer left
        # (B200DEC_A_F16_ROWS16): half the shared memory of converting fp32 rows, so larger tiles fit
        q_kind = nv.A_F16_ROWS16 if (ln and a_kind == nv.A_F16 and kind != nv.W_BF16 and k // s <= 256) else a_kind
        if fits(kind, q_kind, int(ln), w, s, k, max_rows):
            return w, s
    return valid[0]


@dataclass
class PackedLinear:
    kind: int
    n: int
    k: int
    tiled: torch.Tensor
    meta: torch.Tensor | None
    scale: torch.Tensor | None
    bias: torch.Tensor | None
    warps: int
    ksplit: int
    # reference-format operands (kept only when keep_reference=True)
    q: torch.Tensor | None = None
    kept: torch.Tensor | None = None
    words: torch.Tensor | None = None
    # for a projection with a folded LayerNorm: sum_k gamma[k] W[n][k] and sum_k beta[k] W[n][k]
    ln_g: torch.Tensor | None = None
    ln_bias: torch.Tensor | None = None

    def struct(self) -> nv.Weight:
        return nv.Weight(nv.ptr(self.tiled), nv.ptr(self.meta), nv.ptr(self.scale), nv.ptr(self.bias),
                         nv.ptr(self.ln_g), nv.ptr(self.ln_bias), self.n, self.k, self.kind, self.warps, self.ksplit)

    def stream_bytes(self) -> int:
        """Bytes a step reads for this projection: weights (+ selectors) + 4 B scale + bias per channel as stored."""
        b = self.tiled.numel() * self.tiled.element_size()
        if self.meta is not None:
            b += self.meta.numel() * 4
        if self.scale is not None:
            b += self.n * 4
        if self.bias is not None:
            b += self.n * 4
        return b


def pack_linear(weight: torch.Tensor, bias: torch.Tensor | None, kind: int, keep_reference: bool = False, *,
                a_kind: int | None = None, ln: tuple[torch.Tensor, torch.Tensor] | None = None,
                max_rows: int = 64) -> PackedLinear:
    """One (N, K) projection into the streaming layout of the given kind (native.W_BF16 / W_F16 / W_INT8 / W_INT8_24).
    a_kind and max_rows describe how it will be called (operand precision, most rows): they only choose the CTA
    tile. ln = (gamma, beta) of the LayerNorm this projection folds in: the two per-channel vectors of that fold are
    computed here from the weights the kernel multiplies by."""
    w = _f32(weight)
    n, k = w.shape
    lib = nv.lib()
    if a_kind is None:
        a_kind = nv.A_F32_SPLIT if kind == nv.W_BF16 else nv.A_F16
    # the tcgen05 kernels: 128 channels per CTA; the projections split K over a cluster
    if kind in (nv.W_INT8_UMMA, nv.W_F16_UMMA, nv.W_INT8_24_UMMA):
        warps, ksplit = 8, (4 if (k == 1024 and n >= 3072) else 8)  # 96, 128 or 64 CTAs (the head ignores the split)
    else:
        warps, ksplit = tile_config(n, k, kind, a_kind, ln is not None, max_rows)
    ln_g = ln_bias = None
    if ln is not None:
        wd = dequantized(w, kind).double()
        ln_g = (wd @ ln[0].detach().double().to(w.device)).float().contiguous()
        ln_bias = (wd @ ln[1].detach().double().to(w.device)).float().contiguous()
        del wd
    b = None if bias is None else bias.detach().float().contiguous()
    dev = w.device
    tiled = torch.empty(lib.b200dec_tiled_bytes(kind, n, k), dtype=torch.uint8, device=dev)
    meta = scale = q = kept = words = None
    if kind in (nv.W_BF16, nv.W_F16):  # one tiler for both: it moves 16-bit words
        wb = (w.to(torch.bfloat16) if kind == nv.W_BF16 else fp16_image(w)).contiguous()
        nv.check(lib.b200dec_tile_bf16(nv.ptr(wb), n, k, nv.ptr(tiled), nv.stream_ptr()))
    elif kind == nv.W_INT8:
        q, scale = quantize_rows(w)
        nv.check(lib.b200dec_tile_int8(nv.ptr(q), n, k, nv.ptr(tiled), nv.stream_ptr()))
    elif kind == nv.W_F16_UMMA:
        wb = fp16_image(w).contiguous()
        nv.check(lib.b200dec_tile_f16_umma(nv.ptr(wb), n, k, nv.ptr(tiled), nv.stream_ptr()))
    elif kind == nv.W_INT8_UMMA:
        q, scale = quantize_rows(w)
        nv.check(lib.b200dec_tile_int8_umma(nv.ptr(q), n, k, nv.ptr(tiled), nv.stream_ptr()))
    elif kind in (nv.W_INT8_24, nv.W_INT8_24_UMMA):
        q, scale = quantize_rows(prune_24_magnitude(w))
        kept, words = compress_24(q)
        meta = torch.empty(lib.b200dec_tiled_meta_bytes(kind, n, k) // 4, dtype=torch.int32, device=dev)
        tile = lib.b200dec_tile_24 if kind == nv.W_INT8_24 else lib.b200dec_tile_24_umma
        nv.check(tile(nv.ptr(kept), nv.ptr(words), n, k, nv.ptr(tiled), nv.ptr(meta), nv.stream_ptr()))
    else:
        raise ValueError(kind)
    torch.cuda.current_stream().synchronize()  # the temporaries above may be freed once the tilers are done
    if not keep_reference:
        q = kept = words = None
    return PackedLinear(kind, n, k, tiled, meta, scale, b, warps, ksplit, q, kept, words, ln_g, ln_bias)


def fp16_image(w: torch.Tensor) -> torch.Tensor:
    """The fp16 weights of a B200DEC_W_F16 projection: the bf16 value the reference multiplies by
    (server.py:266 loads the model as bf16) rounded to fp16. fp16 has three more mantissa bits than bf16, so every bf16
    value of magnitude 2^-14 .. 65504 is kept exactly; smaller ones land on the fp16 subnormal grid (absolute error
    at most 2^-25), larger ones are refused."""
    wb = w.to(torch.bfloat16).float()
    assert float(wb.abs().max()) <= 65504.0, "a weight beyond the fp16 range: use the bf16 kind"
    return wb.to(torch.float16)


def dequantized(weight: torch.Tensor, kind: int) -> torch.Tensor:
    """fp32 weights the packed projection multiplies by (what an fp32 comparison should use)."""
    w = _f32(weight)
    if kind == nv.W_BF16:
        return w.to(torch.bfloat16).float()
    if kind in (nv.W_F16, nv.W_F16_UMMA):
        return fp16_image(w).float()
    if kind in (nv.W_INT8_24, nv.W_INT8_24_UMMA):
        w = prune_24_magnitude(w)
    q, s = quantize_rows(w)
    return q.float() * s[:, None]
