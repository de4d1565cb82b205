"""Per-kernel parity on a B200, every call through the C-ABI (ctypes): the packers bit-exact against the reference's
outputs (tests/golden/packers.npz) and the numpy oracle, the tiled layouts against their specification, each step
kernel against fp32 numpy on the same seeded inputs."""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import packers as op
from oracle.decoder import activation, bf16_round, layer_norm

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nv():
    from cohere_inference_b200 import native
    native.lib()
    return native


@pytest.fixture(scope="module")
def pk():
    from cohere_inference_b200 import packing
    return packing


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


# ---- packers -----------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("case", ["a", "b", "c"])
def test_packers_bit_exact_vs_reference(pk, golden_dir, case):
    g = np.load(os.path.join(golden_dir, "packers.npz"))
    w = cuda(g[f"{case}_w"])
    u8, s = pk.prepare_w8(w)
    assert np.array_equal(u8.cpu().numpy(), g[f"{case}_u8"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), g[f"{case}_s"].view(np.uint32))
    q, s2 = pk.quantize_rows(w)
    assert np.array_equal(q.cpu().numpy(), op.unpermute_w8(g[f"{case}_u8"])) and torch.equal(s, s2)
    pruned = pk.prune_24_magnitude(w).cpu().numpy()
    rows = np.ones(pruned.shape[0], bool)
    if case == "a":
        rows[[3, 5]] = False  # exact ties: the reference leaves the choice to torch.topk
    assert np.array_equal(pruned[rows], g[f"{case}_pruned"][rows])
    assert np.array_equal(pruned, op.prune_24_magnitude(g[f"{case}_w"]))  # and the documented tie rule everywhere
    kept, words = pk.compress_24(cuda(g[f"{case}_qp"]))
    assert np.array_equal(kept.cpu().numpy(), g[f"{case}_kept"])
    assert np.array_equal(words.cpu().numpy(), g[f"{case}_words"])


def test_compress_patterns_and_rejects_dense(pk, golden_dir):
    g = np.load(os.path.join(golden_dir, "packers.npz"))
    kept, words = pk.compress_24(cuda(g["p_q"]))
    assert np.array_equal(kept.cpu().numpy(), g["p_kept"]) and np.array_equal(words.cpu().numpy(), g["p_words"])
    with pytest.raises(AssertionError):
        pk.compress_24(torch.ones(16, 32, dtype=torch.int8, device="cuda"))


def test_tiled_layouts(nv, pk):
    rng = np.random.default_rng(3)
    n, k = 64, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    # int8: byte [nt][kb][h][lane = 4 g + t][e] = q[16 nt + g + 8 h][64 kb + 16 t + e] + 128
    p = pk.pack_linear(cuda(w), None, nv.W_INT8, keep_reference=True)
    q = p.q.cpu().numpy()
    t = p.tiled.cpu().numpy().reshape(n // 16, k // 64, 2, 8, 4, 16)
    want = (q.astype(np.int16) + 128).astype(np.uint8).reshape(n // 16, 2, 8, k // 64, 4, 16).transpose(0, 3, 1, 2, 4, 5)
    assert np.array_equal(t, want)
    assert np.array_equal(q, op.quantize_rows(w)[0])
    # bf16: element [nt][kb][h][lane][e] = w[16 nt + g + 8 h][32 kb + 8 t + e]
    p = pk.pack_linear(cuda(w), None, nv.W_BF16)
    t = p.tiled.view(torch.bfloat16).float().cpu().numpy().reshape(n // 16, k // 32, 2, 8, 4, 8)
    want = bf16_round(w).reshape(n // 16, 2, 8, k // 32, 4, 8).transpose(0, 3, 1, 2, 4, 5)
    assert np.array_equal(t, want)
    # fp16: the same layout holding fp16(bf16(w)); with these magnitudes every value is the bf16 one exactly
    p = pk.pack_linear(cuda(w), None, nv.W_F16)
    t16 = p.tiled.view(torch.float16).float().cpu().numpy().reshape(n // 16, k // 32, 2, 8, 4, 8)
    big = np.abs(want) >= 2.0 ** -14
    assert np.array_equal(t16[big], want[big]) and np.abs(t16 - want).max() <= 2.0 ** -25
    assert np.array_equal(pk.dequantized(cuda(w), nv.W_F16).cpu().numpy().reshape(n // 16, 2, 8, k // 32, 4, 8)
                          .transpose(0, 3, 1, 2, 4, 5), t16)
    with pytest.raises(AssertionError):
        pk.pack_linear(cuda(w * 1e7), None, nv.W_F16)
    # 2:4 for the tcgen05 kernel: blocks [n / 128][k / 64] of 4 KB kept bytes [half][channel][16] and 256 selector
    # words [half][channel]: a half of a block's k is 32 k = 16 kept bytes = one word of compress_24's row
    w3 = (rng.standard_normal((256, 128)) * 0.02).astype(np.float32)
    p = pk.pack_linear(cuda(w3), None, nv.W_INT8_24_UMMA, keep_reference=True)
    kept3, words3 = p.kept.cpu().numpy(), p.words.cpu().numpy()
    assert np.array_equal(p.tiled.cpu().numpy().view(np.int8).reshape(2, 2, 2, 128, 16),
                          kept3.reshape(2, 128, 2, 2, 16).transpose(0, 2, 3, 1, 4))
    assert np.array_equal(p.meta.cpu().numpy().reshape(2, 2, 2, 128), words3.reshape(2, 128, 2, 2).transpose(0, 2, 3, 1))
    # fp16 for the tcgen05 kernels: blocks [n / 128][k / 64] of 16 KB, each the image of a 128-byte-swizzled K-major
    # tile: channel t's row at 128 t, its 16-byte chunk c at position c ^ (t & 7)
    w2 = (rng.standard_normal((256, 128)) * 0.02).astype(np.float32)
    p = pk.pack_linear(cuda(w2), None, nv.W_F16_UMMA)
    img = pk.fp16_image(cuda(w2)).cpu().numpy()
    tu = p.tiled.view(torch.float16).cpu().numpy().reshape(2, 2, 128, 8, 8)
    tt = np.arange(128)
    for pos in range(8):
        c = pos ^ (tt & 7)  # the chunk that sits at this position of each channel's row
        src = img.reshape(2, 128, 2, 8, 8)[:, tt, :, c, :]  # (t, mt, kb, e)
        assert np.array_equal(tu[:, :, :, pos, :], src.transpose(1, 2, 0, 3))
    # 2:4: value byte [nt][kb][h][lane][2 s + j] = kept[row][2 G + j], G = 32 kb + 2 (4 (s / 2) + t) + (s & 1);
    # selector nibble s of word [nt][kb][h][lane] = the selector of group G
    p = pk.pack_linear(cuda(w), None, nv.W_INT8_24, keep_reference=True)
    kept, words = p.kept.cpu().numpy(), p.words.cpu().numpy().view(np.uint32)
    qd = op.quantize_rows(op.prune_24_magnitude(w))[0]
    k2, w2 = op.compress_24(qd)
    assert np.array_equal(kept, k2) and np.array_equal(words, w2.view(np.uint32))
    tv = p.tiled.cpu().numpy().view(np.int8).reshape(n // 16, k // 128, 2, 8, 4, 8, 2)
    tm = p.meta.cpu().numpy().view(np.uint32).reshape(n // 16, k // 128, 2, 8, 4)
    nib = (words[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 15
    nib = nib.reshape(n, k // 4)
    for nt in range(n // 16):
        for kb in range(k // 128):
            for h in range(2):
                for g in range(8):
                    row = nt * 16 + g + 8 * h
                    for tt in range(4):
                        m = 0
                        for s in range(8):
                            G = kb * 32 + 2 * (4 * (s // 2) + tt) + (s & 1)
                            assert tv[nt, kb, h, g, tt, s, 0] == kept[row, 2 * G]
                            assert tv[nt, kb, h, g, tt, s, 1] == kept[row, 2 * G + 1]
                            m |= int(nib[row, G]) << (4 * s)
                        assert tm[nt, kb, h, g, tt] == m


# ---- projections ---------------------------------------------------------------------------------------------------------

SHAPES = [(3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096), (16384, 1024)]


def _linear_case(nv, pk, kind, a_kind, n, k, rows, act, out_kind, seed, bias=True, ln=False, pdl=0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32) if bias else None
    a = rng.standard_normal((rows, k)).astype(np.float32)
    x0 = rng.standard_normal((rows, n)).astype(np.float32)
    gam = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    bet = (0.1 * rng.standard_normal(k)).astype(np.float32)
    g_d, b_d = cuda(gam), cuda(bet)
    p = pk.pack_linear(cuda(w), None if b is None else cuda(b), kind, a_kind=a_kind, ln=(g_d, b_d) if ln else None,
                       max_rows=rows)
    wd = pk.dequantized(cuda(w), kind).cpu().numpy()
    norm = None
    if ln:  # the operand is LayerNorm(a) of fp32 rows with their own offsets and spreads, folded into the epilogue
        a = (a * (1 + rng.random((rows, 1))) + rng.standard_normal((rows, 1))).astype(np.float32)
        norm = nv.norm(g_d, b_d, 1e-5)
        a_dev = cuda(a)
        a_ref = layer_norm(a, gam, bet, 1e-5)  # exact: the kernel's fp16 rounding of (a - c) * gamma is its error
    elif a_kind == nv.A_F16:
        a_dev = cuda(a.astype(np.float16))
        a_ref = a.astype(np.float16).astype(np.float32)
    else:
        a_dev, a_ref = cuda(a), a
    y = a_ref.astype(np.float64) @ wd.astype(np.float64).T + (0 if b is None else b)
    y = y.astype(np.float32)
    if act != nv.ACT_NONE:
        y = activation({nv.ACT_RELU: "relu", nv.ACT_GELU: "gelu"}[act], y)
    if out_kind == nv.OUT_F16:
        out = torch.zeros(rows, n, dtype=torch.float16, device="cuda")
    else:
        out = cuda(x0) if out_kind == nv.OUT_F32_ADD else torch.zeros(rows, n, device="cuda")
    ws = p.struct()
    nv.check(nv.lib().b200dec_linear(C.byref(ws), nv.ptr(a_dev), a_kind, C.byref(norm) if ln else None, k, rows,
                                     nv.ptr(out), out_kind, n, act, pdl, nv.stream_ptr()))
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    if out_kind == nv.OUT_F32_ADD:
        y = y + x0
    return got, y


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("rows", [1, 8, 13, 64, 128])
def test_linear_int8(nv, pk, n, k, rows):
    got, want = _linear_case(nv, pk, nv.W_INT8, nv.A_F16, n, k, rows, nv.ACT_NONE, nv.OUT_F32, seed=n + rows)
    # operands are exact (fp16 activations given, int8 weights): only the fp32 accumulation order differs
    np.testing.assert_allclose(got, want, atol=2e-4, rtol=1e-5)


@pytest.mark.parametrize("kind,a_kind", [("W_INT8", "A_F32_SPLIT"), ("W_BF16", "A_F32_SPLIT"), ("W_INT8_24", "A_F16"),
                                         ("W_F16", "A_F16"), ("W_F16", "A_F32_SPLIT")])
@pytest.mark.parametrize("n,k", [(1024, 1024), (4096, 1024), (1024, 4096)])
@pytest.mark.parametrize("rows", [3, 64, 100])
def test_linear_kinds(nv, pk, kind, a_kind, n, k, rows):
    got, want = _linear_case(nv, pk, getattr(nv, kind), getattr(nv, a_kind), n, k, rows, nv.ACT_NONE, nv.OUT_F32,
                             seed=7 * n + rows)
    # split operand: ~2^-21 relative on the activations
    np.testing.assert_allclose(got, want, atol=3e-4, rtol=1e-5)


@pytest.mark.parametrize("kind,a_kind", [("W_INT8", "A_F16"), ("W_INT8", "A_F32_SPLIT"), ("W_BF16", "A_F32_SPLIT"),
                                         ("W_INT8_24", "A_F16"), ("W_F16", "A_F16")])
@pytest.mark.parametrize("n", [1024, 3072, 4096])
@pytest.mark.parametrize("rows", [2, 64, 128])
def test_linear_layernorm_on_load(nv, pk, kind, a_kind, n, rows):
    """The operand is LayerNorm(x) of fp32 rows, normalised while staging from statistics the cluster's CTAs exchange."""
    got, want = _linear_case(nv, pk, getattr(nv, kind), getattr(nv, a_kind), n, 1024, rows, nv.ACT_NONE, nv.OUT_F32,
                             seed=3 * n + rows, ln=True)
    # fp16 operand: each of the 1024 terms carries a relative rounding error of up to 2^-11 (outputs are ~0.6 rms);
    # the split operand keeps ~21 bits
    tol = 4e-3 if a_kind == "A_F16" else 4e-4
    np.testing.assert_allclose(got, want, atol=tol, rtol=1e-4)


def _row_sums(x):
    """(rows, 2) float64: sum and sum of squares of every row."""
    return np.stack([x.astype(np.float64).sum(1), (x.astype(np.float64) ** 2).sum(1)], 1)


@pytest.mark.parametrize("kind", ["W_INT8", "W_INT8_24", "W_F16"])
@pytest.mark.parametrize("n", [1024, 3072, 4096])
@pytest.mark.parametrize("rows", [2, 13, 64, 128])
def test_linear_linked_layernorm(nv, pk, kind, n, rows):
    """A projection that updates the residual rows also leaves the next LayerNorm's operand (row * gamma, fp16) and the
    rows' partial sums (one slot per finishing CTA); the LayerNorm-folding projection that stages them equals
    LayerNorm(rows) W^T + b. b200dec_ln_rows16 makes the same pair from fp32 rows."""
    rng = np.random.default_rng(n + rows)
    k = 1024
    wk = getattr(nv, kind)
    lib = nv.lib()
    gam = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    bet = (0.1 * rng.standard_normal(k)).astype(np.float32)
    g_d, b_d = cuda(gam), cuda(bet)
    # producer: x += mid @ Wp^T (a 1024 x 1024 projection)
    wp = (rng.standard_normal((k, k)) * 0.02).astype(np.float32)
    mid = rng.standard_normal((rows, k)).astype(np.float16)
    x0 = (rng.standard_normal((rows, k)) * (1 + rng.random((rows, 1))) + rng.standard_normal((rows, 1))).astype(np.float32)
    pp = pk.pack_linear(cuda(wp), None, nv.W_INT8, max_rows=rows)
    x = cuda(x0)
    x16 = torch.zeros(rows, k, dtype=torch.float16, device="cuda")
    mid_d, ps = cuda(mid), pp.struct()
    slots = lib.b200dec_linear_stat_slots(C.byref(ps))
    sums = torch.full((rows, slots, 2), float("nan"), device="cuda")
    link = nv.LnLink(nv.ptr(g_d), nv.ptr(x16), nv.ptr(sums), None, 0, 0)
    nv.check(lib.b200dec_linear_linked(C.byref(ps), nv.ptr(mid_d), nv.A_F16, None, k, rows, nv.ptr(x), nv.OUT_F32_ADD, k,
                                       nv.ACT_NONE, C.byref(link), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    xn = x.cpu().numpy()
    xw = mid.astype(np.float64) @ pk.dequantized(cuda(wp), nv.W_INT8).cpu().numpy().astype(np.float64).T + x0
    np.testing.assert_allclose(xn, xw.astype(np.float32), atol=2e-4, rtol=1e-5)
    assert np.array_equal(x16.cpu().numpy(), (xn * gam).astype(np.float16)), "the operand is fp16(row * gamma)"
    np.testing.assert_allclose(sums.cpu().numpy().astype(np.float64).sum(1), _row_sums(xn), rtol=1e-5, atol=1e-3)
    # the same pair from fp32 rows: one slot per row
    x16b = torch.zeros_like(x16)
    sums_b = torch.zeros(rows, 2, device="cuda")
    nv.check(lib.b200dec_ln_rows16(nv.ptr(x), nv.ptr(g_d), rows, nv.ptr(x16b), nv.ptr(sums_b), nv.stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(x16b, x16)
    np.testing.assert_allclose(sums_b.cpu().numpy().astype(np.float64), _row_sums(xn), rtol=1e-5, atol=1e-3)
    # reader: LayerNorm folded, operand and sums as left by the producer
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32)
    pc = pk.pack_linear(cuda(w), cuda(b), wk, a_kind=nv.A_F16, ln=(g_d, b_d), max_rows=rows)
    norm, cs = nv.norm(g_d, b_d, 1e-5), pc.struct()
    out = torch.zeros(rows, n, device="cuda")
    for stats, nslots in ((sums, slots), (sums_b, 1)):  # many partials per row, or one
        out.zero_()
        rlink = nv.LnLink(None, None, None, nv.ptr(stats), nslots, 0)
        nv.check(lib.b200dec_linear_linked(C.byref(cs), nv.ptr(x16), nv.A_F16_ROWS16, C.byref(norm), k, rows, nv.ptr(out),
                                           nv.OUT_F32, n, nv.ACT_NONE, C.byref(rlink), 0, nv.stream_ptr()))
        torch.cuda.synchronize()
        want = (layer_norm(xn, gam, bet, 1e-5).astype(np.float64) @
                pk.dequantized(cuda(w), wk).cpu().numpy().astype(np.float64).T + b)
        np.testing.assert_allclose(out.cpu().numpy(), want.astype(np.float32), atol=4e-3, rtol=1e-4)


@pytest.mark.parametrize("offset,atol", [(0.0, 4e-3), (8.0, 8e-3), (32.0, 3e-2)])
@pytest.mark.parametrize("kind", ["W_INT8", "W_INT8_UMMA"])
def test_linked_layernorm_error_grows_with_the_row_offset(nv, pk, offset, atol, kind):
    """The int8 modes stage a row as fp16(row * gamma), unshifted, with plain fp32 sums for the statistics: a row
    whose mean is `offset` standard deviations away from zero loses log2(offset) bits of its deviations to the fp16
    rounding (and the variance E[x^2] - mean^2 loses 2 * log2(offset) of its 24). The bound that is documented, against
    LayerNorm in float64: exact-mode error at offset 0, twice that at 8, under 3e-2 at 32 (outputs are O(1))."""
    rng = np.random.default_rng(int(offset) + 5)
    rows, k, n = 64, 1024, 3072
    lib = nv.lib()
    gam = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    bet = (0.1 * rng.standard_normal(k)).astype(np.float32)
    g_d, b_d = cuda(gam), cuda(bet)
    sign = np.where(rng.random((rows, 1)) < 0.5, -1.0, 1.0)
    x = (rng.standard_normal((rows, k)) + offset * sign).astype(np.float32)
    x_d = cuda(x)
    x16 = torch.zeros(rows, k, dtype=torch.float16, device="cuda")
    sums = torch.zeros(rows, 2, device="cuda")
    nv.check(lib.b200dec_ln_rows16(nv.ptr(x_d), nv.ptr(g_d), rows, nv.ptr(x16), nv.ptr(sums), nv.stream_ptr()))
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32)
    if kind == "W_INT8_UMMA":
        pc = pk.pack_linear(cuda(w), cuda(b), nv.W_INT8_UMMA, ln=(g_d, b_d))
    else:
        pc = pk.pack_linear(cuda(w), cuda(b), nv.W_INT8, a_kind=nv.A_F16, ln=(g_d, b_d), max_rows=rows)
    norm, cs = nv.norm(g_d, b_d, 1e-5), pc.struct()
    out = torch.zeros(rows, n, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rlink = nv.LnLink(None, None, None, nv.ptr(sums), 1, 0, nv.ptr(status))
    nv.check(lib.b200dec_linear_linked(C.byref(cs), nv.ptr(x16), nv.A_F16_ROWS16, C.byref(norm), k, rows, nv.ptr(out),
                                       nv.OUT_F32, n, nv.ACT_NONE, C.byref(rlink), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    wd = pk.dequantized(cuda(w), nv.W_INT8).cpu().numpy().astype(np.float64)
    x64 = x.astype(np.float64)
    ln = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * gam + bet
    want = ln @ wd.T + b
    err = np.abs(out.cpu().numpy() - want).max()
    assert int(status.item()) == 0 and err <= atol, err


@pytest.mark.parametrize("n,act,out_kind", [(3072, "ACT_NONE", "OUT_F32"), (4096, "ACT_GELU", "OUT_F16"),
                                            (1024, "ACT_RELU", "OUT_F32")])
@pytest.mark.parametrize("rows", [1, 13, 64, 100, 128])
@pytest.mark.parametrize("kind", ["W_INT8_UMMA", "W_F16_UMMA", "W_INT8_24_UMMA"])
def test_linear_umma_layernorm(nv, pk, kind, n, act, out_kind, rows):
    """The tcgen05 projection (weight kinds W_INT8_UMMA, and W_F16_UMMA whose tiles come by bulk copy): LayerNorm folded, rows handed over as the ready fp16 operand
    with partial sums; equals act(LayerNorm(rows) W^T + b) on the dequantised weights. Twice in a row (tensor memory
    and the barrier are set up per launch)."""
    rng = np.random.default_rng(n + rows)
    k = 1024
    lib = nv.lib()
    gam = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    bet = (0.1 * rng.standard_normal(k)).astype(np.float32)
    x = (rng.standard_normal((rows, k)) * (1 + rng.random((rows, 1))) + 0.3 * rng.standard_normal((rows, 1))).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32)
    g_d, b_d, x_d = cuda(gam), cuda(bet), cuda(x)
    kind = getattr(nv, kind)
    pc = pk.pack_linear(cuda(w), cuda(b), kind, ln=(g_d, b_d))
    norm, cs = nv.norm(g_d, b_d, 1e-5), pc.struct()
    xg = torch.zeros(rows, k, dtype=torch.float16, device="cuda")
    sums = torch.zeros(rows, 2, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    nv.check(lib.b200dec_ln_rows16(nv.ptr(x_d), nv.ptr(g_d), rows, nv.ptr(xg), nv.ptr(sums), nv.stream_ptr()))
    ok, ak = getattr(nv, out_kind), getattr(nv, act)
    want = layer_norm(x, gam, bet, 1e-5).astype(np.float64) @ pk.dequantized(cuda(w), kind).cpu().numpy().astype(np.float64).T + b
    want = want.astype(np.float32)
    if ak != nv.ACT_NONE:
        want = activation({nv.ACT_RELU: "relu", nv.ACT_GELU: "gelu"}[ak], want)
    link = nv.LnLink(None, None, None, nv.ptr(sums), 1, 0, nv.ptr(status))
    for _ in range(2):
        out = torch.zeros(rows, n, dtype=torch.float16 if ok == nv.OUT_F16 else torch.float32, device="cuda")
        nv.check(lib.b200dec_linear_linked(C.byref(cs), nv.ptr(xg), nv.A_F16_ROWS16, C.byref(norm), k, rows, nv.ptr(out), ok,
                                           n, ak, C.byref(link), 0, nv.stream_ptr()))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        np.testing.assert_allclose(out.float().cpu().numpy(), want, atol=5e-3, rtol=2e-3 if ok == nv.OUT_F16 else 1e-4)


@pytest.mark.parametrize("kind", ["W_INT8_UMMA", "W_INT8", "W_INT8_24", "W_F16", "W_F16_UMMA", "W_INT8_24_UMMA"])
@pytest.mark.parametrize("n,k", [(1024, 1024), (1024, 4096), (3072, 1024)])
@pytest.mark.parametrize("rows", [1, 13, 33, 50, 64, 100, 128])
def test_linear_plain_and_stream_update(nv, pk, kind, n, k, rows):
    """A projection without a LayerNorm (the o, cross-o and fc2 shapes) on the tcgen05 kernel (K split 4 or 8 ways,
    above 64 rows K = 4096 and the 1024-wide shapes as two clusters of 64 rows per tile) and on the mma.sync kernel (fc2 at 33-64 rows: the rows dealt over two CTAs per
    tile): a plain fp32 store, then the residual update that also leaves the next LayerNorm's fp16 operand and
    partial sums."""
    rng = np.random.default_rng(n + k + rows)
    lib = nv.lib()
    kind = getattr(nv, kind)
    a = (rng.standard_normal((rows, k)) * 0.5).astype(np.float16)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32)
    pc = pk.pack_linear(cuda(w), cuda(b), kind)
    cs = pc.struct()
    a_d = cuda(a)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    prod = a.astype(np.float64) @ pk.dequantized(cuda(w), kind).cpu().numpy().astype(np.float64).T + b
    out = torch.zeros(rows, n, device="cuda")
    link = nv.LnLink(None, None, None, None, 0, 0, nv.ptr(status))
    nv.check(lib.b200dec_linear_linked(C.byref(cs), nv.ptr(a_d), nv.A_F16, None, k, rows, nv.ptr(out), nv.OUT_F32, n,
                                       nv.ACT_NONE, C.byref(link), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    np.testing.assert_allclose(out.cpu().numpy(), prod.astype(np.float32), atol=2e-3, rtol=1e-4)
    if n != 1024:
        return
    x0 = rng.standard_normal((rows, n)).astype(np.float32)
    gam = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    g_d = cuda(gam)
    slots = lib.b200dec_linear_stat_slots(C.byref(cs))
    assert kind not in (nv.W_INT8_UMMA, nv.W_F16_UMMA, nv.W_INT8_24_UMMA) or slots == (n // 128) * pc.ksplit
    for _ in range(2):
        x = cuda(x0.copy())
        x16 = torch.zeros(rows, n, dtype=torch.float16, device="cuda")
        sums = torch.full((rows, slots, 2), float("nan"), device="cuda")
        plink = nv.LnLink(nv.ptr(g_d), nv.ptr(x16), nv.ptr(sums), None, 0, 0, nv.ptr(status))
        nv.check(lib.b200dec_linear_linked(C.byref(cs), nv.ptr(a_d), nv.A_F16, None, k, rows, nv.ptr(x), nv.OUT_F32_ADD, n,
                                           nv.ACT_NONE, C.byref(plink), 0, nv.stream_ptr()))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        xn = x.cpu().numpy()
        np.testing.assert_allclose(xn, (x0 + prod).astype(np.float32), atol=2e-3, rtol=1e-4)
        assert torch.equal(x16, (x * g_d).to(torch.float16))
        np.testing.assert_allclose(sums.sum(1).cpu().numpy().astype(np.float64), _row_sums(xn), rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("act", ["ACT_RELU", "ACT_GELU"])
@pytest.mark.parametrize("out_kind", ["OUT_F16", "OUT_F32_ADD"])
def test_linear_epilogues(nv, pk, act, out_kind):
    got, want = _linear_case(nv, pk, nv.W_INT8, nv.A_F16, 4096, 1024, 24, getattr(nv, act), getattr(nv, out_kind), 11)
    tol = 2e-3 if out_kind == "OUT_F16" else 2e-4
    np.testing.assert_allclose(got, want, atol=tol, rtol=1e-3 if out_kind == "OUT_F16" else 1e-5)


def test_linear_no_bias_and_pdl_flag(nv, pk):
    got, want = _linear_case(nv, pk, nv.W_INT8, nv.A_F16, 1024, 1024, 5, nv.ACT_NONE, nv.OUT_F32, 5, bias=False, pdl=1)
    np.testing.assert_allclose(got, want, atol=2e-4, rtol=1e-5)


def test_linear_rejects_bad_arguments(nv, pk):
    p = pk.pack_linear(torch.zeros(1024, 1024, device="cuda"), None, nv.W_INT8)
    ws = p.struct()
    a = torch.zeros(4, 1024, dtype=torch.float16, device="cuda")
    out = torch.zeros(4, 1024, device="cuda")
    rc = nv.lib().b200dec_linear(C.byref(ws), nv.ptr(a), nv.A_F16, None, 1024, 129, nv.ptr(out), nv.OUT_F32, 1024, 0, 0,
                                 nv.stream_ptr())
    assert rc == 1 and b"rows" in nv.lib().b200dec_last_error()
    ws.ksplit = 3
    assert nv.lib().b200dec_linear(C.byref(ws), nv.ptr(a), nv.A_F16, None, 1024, 4, nv.ptr(out), nv.OUT_F32, 1024, 0, 0,
                                   nv.stream_ptr()) == 1
    torch.cuda.synchronize()


@pytest.mark.parametrize("rows", [1, 7, 64, 128])
@pytest.mark.parametrize("a_kind,ln", [("A_F16", False), ("A_F32_SPLIT", False), ("A_F32_SPLIT", True)])
def test_head_argmax(nv, pk, rows, a_kind, ln):
    rng = np.random.default_rng(rows)
    n, k = 16384, 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.01).astype(np.float32)
    a = rng.standard_normal((rows, k)).astype(np.float32)
    gam = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    bet = (0.1 * rng.standard_normal(k)).astype(np.float32)
    g_d, b_d = cuda(gam), cuda(bet)
    p = pk.pack_linear(cuda(w), cuda(b), nv.W_INT8, a_kind=getattr(nv, a_kind), ln=(g_d, b_d) if ln else None,
                       max_rows=rows)
    wd = pk.dequantized(cuda(w), nv.W_INT8).cpu().numpy()
    norm = None
    if ln:
        norm = nv.norm(g_d, b_d, 1e-5)
        a_dev, a_ref = cuda(a), layer_norm(a, gam, bet, 1e-5)
    elif a_kind == "A_F16":
        a_dev, a_ref = cuda(a.astype(np.float16)), a.astype(np.float16).astype(np.float32)
    else:
        a_dev, a_ref = cuda(a), a
    ws = p.struct()
    np_ = nv.lib().b200dec_head_partials(C.byref(ws))
    pm = torch.zeros(rows, np_, device="cuda")
    pi = torch.zeros(rows, np_, dtype=torch.int32, device="cuda")
    logits = torch.zeros(rows, n, device="cuda")
    nv.check(nv.lib().b200dec_head_argmax(C.byref(ws), nv.ptr(a_dev), getattr(nv, a_kind), C.byref(norm) if ln else None,
                                          k, rows, nv.ptr(pm), nv.ptr(pi), nv.ptr(logits), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    want = (a_ref.astype(np.float64) @ wd.astype(np.float64).T + b).astype(np.float32)
    lg = logits.cpu().numpy()
    np.testing.assert_allclose(lg, want, atol=4e-4, rtol=1e-5)
    # the partials are exactly the first-index maxima of the kernel's own logits, tile by tile
    tile = n // np_
    t = lg.reshape(rows, np_, tile)
    assert np.array_equal(pm.cpu().numpy(), t.max(-1))
    assert np.array_equal(pi.cpu().numpy(), t.argmax(-1) + np.arange(np_) * tile)


@pytest.mark.parametrize("rows", [1, 33, 64, 100])
@pytest.mark.parametrize("n", [256, 16384])
@pytest.mark.parametrize("kind", ["W_INT8_UMMA", "W_F16_UMMA"])
def test_head_umma(nv, pk, kind, rows, n):
    """The tcgen05 vocabulary projection: logits vs fp64 on the dequantised weights (operand fp16, so the tolerance of
    the other fp16-operand projections), partials = first-index maxima of its own logits per 128 channels; twice in a
    row (tensor memory and barriers are set up per launch)."""
    rng = np.random.default_rng(rows + n)
    k = 1024
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(n) * 0.01).astype(np.float32)
    a = (rng.standard_normal((rows, k)) * 1.5 + 0.3).astype(np.float32)
    gam = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    bet = (0.1 * rng.standard_normal(k)).astype(np.float32)
    g_d, b_d, a_d = cuda(gam), cuda(bet), cuda(a)
    kind = getattr(nv, kind)
    p = pk.pack_linear(cuda(w), cuda(b), kind)
    wd = pk.dequantized(cuda(w), kind).cpu().numpy()
    norm, ws = nv.norm(g_d, b_d, 1e-5), p.struct()
    np_ = nv.lib().b200dec_head_partials(C.byref(ws))
    assert np_ == n // 128
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if kind == nv.W_F16_UMMA:  # fp16 weight tiles go with the ready fp16 operand only: fp32 rows are refused
        pm = torch.zeros(rows, np_, device="cuda")
        pi = torch.zeros(rows, np_, dtype=torch.int32, device="cuda")
        rc = nv.lib().b200dec_head_umma(C.byref(ws), nv.ptr(a_d), C.byref(norm), k, rows, nv.ptr(pm), nv.ptr(pi), None,
                                        nv.ptr(status), 0, nv.stream_ptr())
        assert rc == 1  # B200DEC_EINVAL
    for _ in range(0 if kind == nv.W_F16_UMMA else 2):
        pm = torch.full((rows, np_), -7.0, device="cuda")
        pi = torch.full((rows, np_), -7, dtype=torch.int32, device="cuda")
        logits = torch.zeros(rows, n, device="cuda")
        nv.check(nv.lib().b200dec_head_umma(C.byref(ws), nv.ptr(a_d), C.byref(norm), k, rows, nv.ptr(pm), nv.ptr(pi),
                                            nv.ptr(logits), nv.ptr(status), 0, nv.stream_ptr()))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        a_ref = layer_norm(a, gam, bet, 1e-5).astype(np.float16).astype(np.float64)
        want = (a_ref @ wd.astype(np.float64).T + b).astype(np.float32)
        lg = logits.cpu().numpy()
        np.testing.assert_allclose(lg, want, atol=4e-4, rtol=1e-5)
        t = lg.reshape(rows, np_, 128)
        assert np.array_equal(pm.cpu().numpy(), t.max(-1))
        assert np.array_equal(pi.cpu().numpy(), t.argmax(-1) + np.arange(np_) * 128)
    # the same rows handed over as the ready fp16 operand (row * gamma) with their sums: LayerNorm folded into the epilogue
    pl = pk.pack_linear(cuda(w), cuda(b), kind, ln=(g_d, b_d))
    wl = pl.struct()
    xg = torch.zeros(rows, k, dtype=torch.float16, device="cuda")
    sums = torch.zeros(rows, 2, device="cuda")
    nv.check(nv.lib().b200dec_ln_rows16(nv.ptr(a_d), nv.ptr(g_d), rows, nv.ptr(xg), nv.ptr(sums), nv.stream_ptr()))
    pm = torch.full((rows, np_), -7.0, device="cuda")
    pi = torch.full((rows, np_), -7, dtype=torch.int32, device="cuda")
    logits = torch.zeros(rows, n, device="cuda")
    nv.check(nv.lib().b200dec_head_umma_linked(C.byref(wl), nv.ptr(xg), nv.ptr(sums), 1, C.byref(norm), k, rows,
                                               nv.ptr(pm), nv.ptr(pi), nv.ptr(logits), nv.ptr(status), 0,
                                               nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = (layer_norm(a, gam, bet, 1e-5).astype(np.float64) @ wd.astype(np.float64).T + b).astype(np.float32)
    lg = logits.cpu().numpy()
    np.testing.assert_allclose(lg, want, atol=4e-3, rtol=1e-4)
    t = lg.reshape(rows, np_, 128)
    assert np.array_equal(pm.cpu().numpy(), t.max(-1))
    assert np.array_equal(pi.cpu().numpy(), t.argmax(-1) + np.arange(np_) * 128)


# ---- row kernels ---------------------------------------------------------------------------------------------------------

def test_embed_ln_and_layer_norm(nv):
    rng = np.random.default_rng(5)
    vocab, max_pos, S, rows = 512, 64, 6, 5
    emb = bf16_round((rng.standard_normal((vocab, 1024)) * 0.02).astype(np.float32))
    ptab = bf16_round((rng.standard_normal((max_pos, 1024)) * 0.02).astype(np.float32))
    lnp = [(1 + 0.1 * rng.standard_normal(1024)).astype(np.float32) if i % 2 == 0 else
           (0.1 * rng.standard_normal(1024)).astype(np.float32) for i in range(4)]
    active = np.array([3, 0, 6, 5, 1], np.int32)
    tok = rng.integers(0, vocab, S + 1).astype(np.int64)
    pos = rng.integers(0, max_pos, S + 1).astype(np.int32)
    d = {k: cuda(v) for k, v in dict(w0=lnp[0], b0=lnp[1], w1=lnp[2], b1=lnp[3]).items()}
    x = torch.zeros(rows, 1024, device="cuda")
    hn = torch.zeros(rows, 1024, dtype=torch.float16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # every device operand is held in a variable until the synchronize: a temporary would be freed (and its block
    # reused by the next allocation) before the asynchronous kernel reads it
    a_d, t_d, p_d = cuda(active), cuda(tok), cuda(pos)
    e_d, pt_d = cuda(emb).to(torch.bfloat16), cuda(ptab).to(torch.bfloat16)
    nv.check(nv.lib().b200dec_embed_ln(nv.ptr(a_d), nv.ptr(t_d), nv.ptr(p_d), nv.ptr(e_d), nv.ptr(pt_d), vocab,
                                       max_pos, S, nv.norm(d["w0"], d["b0"], 1e-5), nv.norm(d["w1"], d["b1"], 1e-5),
                                       nv.ptr(x), nv.ptr(hn), nv.OUT_F16, rows, nv.ptr(status), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    want_x = layer_norm(emb[tok[active]] + ptab[pos[active]], lnp[0], lnp[1], 1e-5)
    want_h = layer_norm(want_x, lnp[2], lnp[3], 1e-5)
    np.testing.assert_allclose(x.cpu().numpy(), want_x, atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(hn.float().cpu().numpy(), want_h, atol=3e-3, rtol=1e-3)
    assert int(status.item()) == 0
    h32 = torch.zeros(rows, 1024, device="cuda")
    nv.check(nv.lib().b200dec_layer_norm(nv.ptr(x), nv.norm(d["w1"], d["b1"], 1e-5), nv.ptr(h32), nv.OUT_F32, rows, 0,
                                         nv.stream_ptr()))
    torch.cuda.synchronize()
    np.testing.assert_allclose(h32.cpu().numpy(), layer_norm(x.cpu().numpy(), lnp[2], lnp[3], 1e-5), atol=2e-5, rtol=1e-5)


def test_embed_out_of_range_sets_status_not_a_fault(nv):
    """A token id or position outside its table is clamped and reported through the status word."""
    emb = torch.zeros(16, 1024, dtype=torch.bfloat16, device="cuda")
    ones, zeros = torch.ones(1024, device="cuda"), torch.zeros(1024, device="cuda")
    x = torch.zeros(1, 1024, device="cuda")
    hn = torch.zeros(1, 1024, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    n = nv.norm(ones, zeros, 1e-5)
    active = torch.tensor([0, 7], dtype=torch.int32, device="cuda")  # slot 7 is outside the 0..2 table
    tok = torch.tensor([99, 0, 0], device="cuda")
    pos = torch.tensor([77, 0, 0], dtype=torch.int32, device="cuda")
    x = torch.zeros(2, 1024, device="cuda")
    hn = torch.zeros(2, 1024, device="cuda")
    nv.check(nv.lib().b200dec_embed_ln(nv.ptr(active), nv.ptr(tok), nv.ptr(pos), nv.ptr(emb), nv.ptr(emb), 16, 16, 2,
                                       n, n, nv.ptr(x), nv.ptr(hn), nv.OUT_F32, 2, nv.ptr(status), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == nv.ST_TOKEN_RANGE | nv.ST_POS_RANGE | nv.ST_SLOT_RANGE


def _attention_ref(q, k, v, scale):
    s = (k.astype(np.float64) @ q.astype(np.float64)) * scale
    p = np.exp(s - s.max())
    p /= p.sum()
    return (p @ v.astype(np.float64)).astype(np.float32)


@pytest.mark.parametrize("H,D", [(16, 64), (8, 128)])
@pytest.mark.parametrize("rows", [1, 5, 41, 64])  # 41 and 64 rows x 16 heads: the long-with-short paired kernel (odd, even)
@pytest.mark.parametrize("self_", [0, 1])
@pytest.mark.parametrize("cap", [96, 300])  # one span of keys per row, and several (partials merged in order)
@pytest.mark.parametrize("ring", [False, True])  # the one-CTA-per-(row, head) kernel and the persistent ring kernel
def test_attention(nv, H, D, rows, self_, cap, ring):
    rng = np.random.default_rng(rows * 10 + H + self_ + cap)
    S = max(rows, 4) + 2
    kc = bf16_round(rng.standard_normal((S + 1, H, cap, D)).astype(np.float32))
    vc = bf16_round(rng.standard_normal((S + 1, H, cap, D)).astype(np.float32))
    active = rng.permutation(S)[:rows].astype(np.int32)
    n = rng.integers(0 if self_ else 1, cap - 1, S + 1).astype(np.int32)
    n[active[0]] = 0 if self_ else 1  # shortest case
    if rows > 1:
        n[active[1]] = cap - 1 if self_ else cap  # longest case
    if rows >= 5 and cap > 130:
        n[active[2]], n[active[3]], n[active[4]] = 128, 129, 256  # span boundaries
    if rows == 41:
        n[active[5:20]] = 77  # many equal lengths: pairs that skip the exchange, ties in the ranking
    ld = 3 * H * D if self_ else H * D
    q = rng.standard_normal((rows, ld)).astype(np.float32)
    kd, vd = cuda(kc).to(torch.bfloat16), cuda(vc).to(torch.bfloat16)
    lib = nv.lib()
    part = torch.zeros(lib.b200dec_attention_scratch_floats(rows, H, D), device="cuda")
    count = torch.zeros(rows * H, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(rows, H * D, device="cuda")
    scale = D ** -0.5
    a_d, q_d, n_d = cuda(active), cuda(q), cuda(n)  # held until the synchronize
    for _ in range(2):  # twice: the split counters must have been reset
        fn = lib.b200dec_attention_ring if ring else lib.b200dec_attention
        nv.check(fn(self_, nv.ptr(a_d), nv.ptr(q_d), ld, nv.ptr(kd), nv.ptr(vd), nv.ptr(n_d), S, H, D, cap, scale,
                    nv.ptr(out), nv.OUT_F32, rows, nv.ptr(part), nv.ptr(count), nv.ptr(status), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(count.abs().sum().item()) == 0
    got = out.cpu().numpy()
    k_after = kd.float().cpu().numpy()
    for r in range(rows):
        s = active[r]
        for h in range(H):
            qq = q[r, h * D:(h + 1) * D]
            if self_:
                kn = bf16_round(q[r, (H + h) * D:(H + h + 1) * D])
                vn = bf16_round(q[r, (2 * H + h) * D:(2 * H + h + 1) * D])
                assert np.array_equal(k_after[s, h, n[s]], kn)
                K = np.concatenate([kc[s, h, :n[s]], kn[None]])
                V = np.concatenate([vc[s, h, :n[s]], vn[None]])
            else:
                K, V = kc[s, h, :n[s]], vc[s, h, :n[s]]
            np.testing.assert_allclose(got[r, h * D:(h + 1) * D], _attention_ref(qq, K, V, scale), atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("H,D", [(16, 64), (8, 128)])
@pytest.mark.parametrize("rows", [2, 41, 64])
@pytest.mark.parametrize("self_", [0, 1])
def test_row_schedule_and_paired_attention(nv, H, D, rows, self_):
    """The schedule is the rows by decreasing length (ties by row) with their slots; the paired kernel driven by it
    equals the reference attention and appends the new keys, twice in a row."""
    cap = 300
    rng = np.random.default_rng(rows + H + self_)
    S = rows + 3
    kc = bf16_round(rng.standard_normal((S + 1, H, cap, D)).astype(np.float32))
    vc = bf16_round(rng.standard_normal((S + 1, H, cap, D)).astype(np.float32))
    active = rng.permutation(S)[:rows].astype(np.int32)
    n = rng.integers(0 if self_ else 1, cap - 1, S + 1).astype(np.int32)
    n[active[0]] = 0 if self_ else 1
    n[active[1]] = cap - 1 if self_ else cap
    if rows > 20:
        n[active[5:20]] = 77                       # ties, and pairs of equal length (no exchange)
        n[active[20]], n[active[21]] = 100, 131    # a difference just under / over the exchange threshold
    ld = 3 * H * D if self_ else H * D
    q = rng.standard_normal((rows, ld)).astype(np.float32)
    kd, vd = cuda(kc).to(torch.bfloat16), cuda(vc).to(torch.bfloat16)
    lib = nv.lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sched = torch.full((rows, 4), -1, dtype=torch.int32, device="cuda")
    out = torch.zeros(rows, H * D, device="cuda")
    a_d, q_d, n_d = cuda(active), cuda(q), cuda(n)
    scale = D ** -0.5
    for _ in range(2):
        nv.check(lib.b200dec_row_schedule(nv.ptr(a_d), nv.ptr(n_d) if self_ else None, None if self_ else nv.ptr(n_d), S,
                                          cap, cap, rows, 0, nv.ptr(sched) if self_ else None,
                                          None if self_ else nv.ptr(sched), nv.ptr(status), nv.stream_ptr()))
        nv.check(lib.b200dec_attention_paired(self_, nv.ptr(sched), nv.ptr(q_d), ld, nv.ptr(kd), nv.ptr(vd), H, D, cap,
                                              scale, nv.ptr(out), nv.OUT_F32, rows, 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    lens = n[active]
    order = sorted(range(rows), key=lambda r: (-int(lens[r]), r))
    want = np.array([[r, active[r], lens[r], 0] for r in order], np.int32)
    np.testing.assert_array_equal(sched.cpu().numpy(), want)
    got, k_after = out.cpu().numpy(), kd.float().cpu().numpy()
    for r in range(rows):
        s = active[r]
        for h in range(H):
            qq = q[r, h * D:(h + 1) * D]
            if self_:
                kn = bf16_round(q[r, (H + h) * D:(H + h + 1) * D])
                vn = bf16_round(q[r, (2 * H + h) * D:(2 * H + h + 1) * D])
                assert np.array_equal(k_after[s, h, n[s]], kn)
                K = np.concatenate([kc[s, h, :n[s]], kn[None]])
                V = np.concatenate([vc[s, h, :n[s]], vn[None]])
            else:
                K, V = kc[s, h, :n[s]], vc[s, h, :n[s]]
            np.testing.assert_allclose(got[r, h * D:(h + 1) * D], _attention_ref(qq, K, V, scale), atol=2e-5, rtol=1e-4)


def test_row_schedule_reports_bad_state(nv):
    lib = nv.lib()
    active = cuda(np.array([0, 9, 1], np.int32))          # slot 9 does not exist (slots = 3)
    lens = cuda(np.array([5, 400, 7, 1], np.int32))        # 400 frames > the capacity of 100
    sched = torch.zeros(3, 4, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    nv.check(lib.b200dec_row_schedule(nv.ptr(active), None, nv.ptr(lens), 3, 100, 100, 3, 0, None, nv.ptr(sched),
                                      nv.ptr(status), nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == nv.ST_SLOT_RANGE | nv.ST_FRAMES_RANGE
    np.testing.assert_array_equal(sched.cpu().numpy(), [[2, 1, 100, 0], [0, 0, 5, 0], [1, 3, 1, 0]])


def _kv8(a):
    from oracle.decoder import kv_int8
    return kv_int8(bf16_round(a))


@pytest.mark.parametrize("H,D", [(16, 64), (8, 128)])
def test_scatter_kv_q8_bit_exact(nv, H, D):
    """int8 cross caches and their scales equal the quantiser of the reference's int8 mode applied to the bf16-rounded
    vectors, bit for bit (incl. an all-zero vector: scale 1)."""
    rng = np.random.default_rng(D)
    L, S1, T, rows = 3, 4, 7, 9
    kv = (rng.standard_normal((rows, L * 2 * H * D)) * rng.uniform(0.01, 30, (rows, 1))).astype(np.float32)
    kv[2, :D] = 0.0
    slot_of = rng.integers(0, S1, rows).astype(np.int32)
    frame_of = np.arange(rows, dtype=np.int32) % T
    (slot_of[7], frame_of[7]), (slot_of[8], frame_of[8]) = (1, 0), (2, 0)  # distinct (slot, frame) pairs
    pairs = set()
    for i in range(rows):
        while (slot_of[i], frame_of[i]) in pairs:
            frame_of[i] = (frame_of[i] + 1) % T
        pairs.add((slot_of[i], frame_of[i]))
    ck = torch.zeros(L, S1, H, T, D, dtype=torch.int8, device="cuda")
    cv = torch.zeros_like(ck)
    cks = torch.full((L, S1, H, T), -1.0, device="cuda")
    cvs = torch.full_like(cks, -1.0)
    kv_d, so_d, fo_d = cuda(kv), cuda(slot_of), cuda(frame_of)
    nv.check(nv.lib().b200dec_scatter_kv_q8(nv.ptr(kv_d), nv.ptr(so_d), nv.ptr(fo_d), nv.ptr(ck), nv.ptr(cv), nv.ptr(cks),
                                            nv.ptr(cvs), rows, L, S1, H, D, T, nv.stream_ptr()))
    torch.cuda.synchronize()
    x = kv.reshape(rows, L, 2, H, D)
    for i in range(rows):
        for which, (c, cs) in enumerate(((ck, cks), (cv, cvs))):
            q, sc = _kv8(x[i, :, which])  # (L, H, D), (L, H, 1)
            assert np.array_equal(c[:, slot_of[i], :, frame_of[i]].cpu().numpy(), q)
            assert np.array_equal(cs[:, slot_of[i], :, frame_of[i]].cpu().numpy(), sc[..., 0])


@pytest.mark.parametrize("H,D", [(16, 64), (8, 128)])
@pytest.mark.parametrize("rows", [3, 41])   # one CTA per (row, head, split); rows paired in clusters
@pytest.mark.parametrize("self_", [0, 1])
@pytest.mark.parametrize("paired", [False, True])
def test_attention_q8(nv, H, D, rows, self_, paired):
    """Attention over int8 caches vs fp64 on the dequantised caches; the appended key and value are stored in the
    reference's int8 form (bit-exact) and attended in this step as their bf16 values."""
    if paired and rows < 41:
        pytest.skip("the schedule-driven kernel is for large batches")
    cap = 200
    rng = np.random.default_rng(rows + H + self_)
    S = rows + 2
    kq = rng.integers(-127, 128, (S + 1, H, cap, D)).astype(np.int8)
    vq = rng.integers(-127, 128, (S + 1, H, cap, D)).astype(np.int8)
    ksc = rng.uniform(0.002, 0.03, (S + 1, H, cap)).astype(np.float32)
    vsc = rng.uniform(0.002, 0.03, (S + 1, H, cap)).astype(np.float32)
    active = rng.permutation(S)[:rows].astype(np.int32)
    n = rng.integers(0 if self_ else 1, cap - 1, S + 1).astype(np.int32)
    n[active[0]] = 0 if self_ else 1
    n[active[1]] = cap - 1 if self_ else cap
    ld = 3 * H * D if self_ else H * D
    q = rng.standard_normal((rows, ld)).astype(np.float32)
    kd, vd, ksd, vsd = cuda(kq), cuda(vq), cuda(ksc), cuda(vsc)
    lib = nv.lib()
    part = torch.zeros(lib.b200dec_attention_scratch_floats(rows, H, D), device="cuda")
    count = torch.zeros(rows * H, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sched = torch.zeros(rows, 4, dtype=torch.int32, device="cuda")
    out = torch.zeros(rows, H * D, device="cuda")
    scale = D ** -0.5
    a_d, q_d, n_d = cuda(active), cuda(q), cuda(n)
    if paired:
        nv.check(lib.b200dec_row_schedule(nv.ptr(a_d), nv.ptr(n_d) if self_ else None, None if self_ else nv.ptr(n_d), S,
                                          cap, cap, rows, 0, nv.ptr(sched) if self_ else None,
                                          None if self_ else nv.ptr(sched), nv.ptr(status), nv.stream_ptr()))
        nv.check(lib.b200dec_attention_paired_q8(self_, nv.ptr(sched), nv.ptr(q_d), ld, nv.ptr(kd), nv.ptr(vd), nv.ptr(ksd),
                                                 nv.ptr(vsd), H, D, cap, scale, nv.ptr(out), nv.OUT_F32, rows, 0,
                                                 nv.stream_ptr()))
    else:
        nv.check(lib.b200dec_attention_q8(self_, nv.ptr(a_d), nv.ptr(q_d), ld, nv.ptr(kd), nv.ptr(vd), nv.ptr(ksd),
                                          nv.ptr(vsd), nv.ptr(n_d), S, H, D, cap, scale, nv.ptr(out), nv.OUT_F32, rows,
                                          nv.ptr(part), nv.ptr(count), nv.ptr(status), 0, nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(count.abs().sum().item()) == 0
    got = out.cpu().numpy()
    k_after, ks_after = kd.cpu().numpy(), ksd.cpu().numpy()
    v_after, vs_after = vd.cpu().numpy(), vsd.cpu().numpy()
    kf = kq.astype(np.float32) * ksc[..., None]
    vf = vq.astype(np.float32) * vsc[..., None]
    for r in range(rows):
        s = active[r]
        for h in range(H):
            qq = q[r, h * D:(h + 1) * D]
            if self_:
                kn = bf16_round(q[r, (H + h) * D:(H + h + 1) * D])
                vn = bf16_round(q[r, (2 * H + h) * D:(2 * H + h + 1) * D])
                (kq8, ks8), (vq8, vs8) = _kv8(kn), _kv8(vn)
                assert np.array_equal(k_after[s, h, n[s]], kq8) and ks_after[s, h, n[s]] == ks8[0]
                assert np.array_equal(v_after[s, h, n[s]], vq8) and vs_after[s, h, n[s]] == vs8[0]
                K = np.concatenate([kf[s, h, :n[s]], kn[None]])
                V = np.concatenate([vf[s, h, :n[s]], vn[None]])
            else:
                K, V = kf[s, h, :n[s]], vf[s, h, :n[s]]
            # the int8 pass multiplies in fp16 pairs (exact int8 -> fp16, query and softmax weights rounded to fp16):
            # about 1e-3 relative, well below the int8 rounding of real caches
            np.testing.assert_allclose(got[r, h * D:(h + 1) * D], _attention_ref(qq, K, V, scale), atol=4e-3, rtol=2e-3)


def test_pick_semantics(nv):
    """dec_pick's bookkeeping: forced prompt tokens, greedy after it, end at eos or the limit, dummy and finished rows
    untouched, ties to the lowest index."""
    S, P, cols, np_ = 5, 4, 12, 8
    active = np.array([0, 1, 2, 5, 3], np.int32)  # 5 = dummy
    pm = np.full((5, np_), -1.0, np.float32)
    pi = np.tile(np.arange(np_, dtype=np.int32) * 10, (5, 1))
    pm[0, 3] = 2.0                       # slot 0: inside the prompt -> forced token wins
    pm[1, 2] = pm[1, 6] = 1.5            # slot 1: tie -> index 20
    pm[2, 7] = 9.0                       # slot 2: argmax 70 = eos -> finished
    pm[4, 1] = 3.0                       # slot 3: already finished -> untouched
    pos = np.array([0, 3, 5, 7, 2, 0], np.int32)
    plen = np.array([3, 2, 2, 2, 2, 1], np.int32)
    limit = np.array([9, 4, 9, 9, 9, 0], np.int32)
    fin = np.array([0, 0, 0, 1, 0, 1], np.uint8)
    forced = np.arange((S + 1) * P, dtype=np.int64).reshape(S + 1, P) + 100
    d = {k: cuda(v) for k, v in dict(pm=pm, pi=pi, active=active, pos=pos, plen=plen, limit=limit, fin=fin,
                                     forced=forced).items()}
    tok = torch.zeros(S + 1, dtype=torch.long, device="cuda")
    out = torch.full((S + 1, cols), -1, dtype=torch.long, device="cuda")
    arg = torch.full((S + 1,), -1, dtype=torch.long, device="cuda")
    host_flags = torch.full((S + 1,), 9, dtype=torch.uint8).pin_memory()
    nv.check(nv.lib().b200dec_pick(nv.ptr(d["pm"]), nv.ptr(d["pi"]), np_, nv.ptr(d["active"]), 5, S, nv.ptr(tok),
                                   nv.ptr(d["pos"]), nv.ptr(d["fin"]), nv.ptr(d["forced"]), P, nv.ptr(d["plen"]),
                                   nv.ptr(d["limit"]), nv.ptr(out), cols, 70, nv.ptr(arg), host_flags.data_ptr(), 0,
                                   nv.stream_ptr()))
    torch.cuda.synchronize()
    # a row that ends at this step sets its slot's byte in pinned host memory (written by the kernel itself); rows
    # that go on, rows that ended earlier and the dummy write nothing
    assert host_flags.numpy().tolist() == [9, 1, 1, 9, 9, 9]
    tok, out, arg = tok.cpu().numpy(), out.cpu().numpy(), arg.cpu().numpy()
    pos2, fin2 = d["pos"].cpu().numpy(), d["fin"].cpu().numpy()
    assert (tok[0], pos2[0], fin2[0], out[0, 1], arg[0]) == (101, 1, 0, 101, 30)
    assert (tok[1], pos2[1], fin2[1], out[1, 4], arg[1]) == (20, 4, 1, 20, 20)      # limit reached
    assert (tok[2], pos2[2], fin2[2], out[2, 6]) == (70, 6, 1, 70)                  # eos
    assert (tok[3], pos2[3], fin2[3]) == (0, 7, 1) and (out[3] == -1).all()         # finished: untouched
    assert (pos2[5], fin2[5]) == (0, 1) and arg[5] == -1                             # dummy: untouched


def test_scatter_kv(nv):
    rng = np.random.default_rng(9)
    L, S1, H, D, T = 2, 4, 16, 64, 10
    lengths, slots = [3, 10, 1], [2, 0, 3]
    kv = rng.standard_normal((sum(lengths), L * 2 * H * D)).astype(np.float32)
    slot_of = np.repeat(np.array(slots, np.int32), lengths)
    frame_of = np.concatenate([np.arange(n, dtype=np.int32) for n in lengths])
    ck = torch.zeros(L, S1, H, T, D, dtype=torch.bfloat16, device="cuda")
    cv = torch.zeros_like(ck)
    kv_d, so_d, fo_d = cuda(kv), cuda(slot_of), cuda(frame_of)  # held until the synchronize
    nv.check(nv.lib().b200dec_scatter_kv(nv.ptr(kv_d), nv.ptr(so_d), nv.ptr(fo_d), nv.ptr(ck),
                                         nv.ptr(cv), kv.shape[0], L, S1, H, D, T, nv.stream_ptr()))
    torch.cuda.synchronize()
    want_k, want_v = np.zeros((L, S1, H, T, D), np.float32), np.zeros((L, S1, H, T, D), np.float32)
    r = bf16_round(kv).reshape(-1, L, 2, H, D)
    for i in range(kv.shape[0]):
        want_k[:, slot_of[i], :, frame_of[i]] = r[i, :, 0]
        want_v[:, slot_of[i], :, frame_of[i]] = r[i, :, 1]
    assert np.array_equal(ck.float().cpu().numpy(), want_k) and np.array_equal(cv.float().cpu().numpy(), want_v)


# ---- cross-attention prefill: the tcgen05 GEMM with the cache scatter as its epilogue ---------------------------------

def _image_rows(img, m, k):
    """Decode an operand image (csrc/prefill_gemm.cu) back to (m, k) fp32 = high + low bf16 halves."""
    raw = img.view(torch.int16).cpu().numpy().view(np.uint16)
    r, c = np.meshgrid(np.arange(m), np.arange(k), indexing="ij")
    nkb = k // 64

    def at(block):  # uint16 index of element (r, c) in the given k-block of its row tile
        rr, chunk = r % 128, (c % 64) // 8
        off = (rr >> 3) * 1024 + (rr & 7) * 128 + ((chunk ^ (rr & 7)) << 4) + (c % 8) * 2
        return (((r // 128) * (2 * nkb) + block) * 16384 + off) // 2
    hi = raw[at(c // 64)].astype(np.uint32) << 16
    lo = raw[at(nkb + c // 64)].astype(np.uint32) << 16
    return hi.view(np.float32).astype(np.float64) + lo.view(np.float32).astype(np.float64)


def _prefill_setup(nv, m, k, n, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = bf16_round((rng.standard_normal((n, k)) * 0.03).astype(np.float32))
    b = rng.standard_normal(n).astype(np.float32)
    lib = nv.lib()
    wimg = torch.empty(n * k * 2, dtype=torch.uint8, device="cuda")
    w_d = cuda(w).to(torch.bfloat16)
    nv.check(lib.b200dec_prefill_tile_weight(nv.ptr(w_d), n, k, nv.ptr(wimg), nv.stream_ptr()))
    ximg = torch.zeros(lib.b200dec_prefill_rows_bytes(m, k), dtype=torch.uint8, device="cuda")
    assert ximg.data_ptr() % 1024 == 0 and wimg.data_ptr() % 1024 == 0
    x_d = cuda(x)  # device copies are kept in variables: a temporary would be freed (and its memory reused) at once
    nv.check(lib.b200dec_prefill_pack_rows(nv.ptr(x_d), m, k, k, nv.ptr(ximg), nv.stream_ptr()))
    torch.cuda.synchronize()
    want = x.astype(np.float64) @ w.astype(np.float64).T + b
    return x, w, cuda(b), ximg, wimg, want


@pytest.mark.parametrize("m,k,n", [(301, 1024, 512), (128, 1280, 256), (1000, 64, 1024)])
def test_prefill_gemm_operand_image(nv, m, k, n):
    """mode 0: rows x weights^T + bias, handed on as the next product's operand (two bf16 halves): fp32-level accuracy."""
    x, w, b_d, ximg, wimg, want = _prefill_setup(nv, m, k, n, 3)
    np.testing.assert_allclose(_image_rows(ximg, m, k), x, atol=0, rtol=2.0 ** -16)  # the split keeps ~16 bits
    lib = nv.lib()
    out = torch.zeros(lib.b200dec_prefill_rows_bytes(m, n), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):
        nv.check(lib.b200dec_prefill_gemm(nv.ptr(ximg), m, k, nv.ptr(wimg), nv.ptr(b_d), n, 0, nv.ptr(out), None, 0,
                                          None, None, None, None, 0, 0, 0, 0, 0, nv.ptr(status), nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = _image_rows(out, m, n)
    np.testing.assert_allclose(got, want, atol=2e-4 * np.sqrt(k / 1024), rtol=3e-5)


@pytest.mark.parametrize("H,D,q8", [(4, 64, False), (2, 128, False), (4, 64, True), (2, 128, True)])
def test_prefill_gemm_cache_epilogue(nv, H, D, q8):
    """modes 1 / 2: the product written straight into the slot caches by (piece -> slot, frame); untouched cache cells
    keep their contents; int8 caches hold what the reference's quantiser makes of the bf16-rounded values."""
    L, S1, T, k = 2, 5, 160, 1024
    n = L * 2 * H * D
    pieces = np.array([[0, 100, 3, 0], [100, 160, 0, 0], [260, 41, 4, 0]], np.int32)
    m = 301
    x, w, b_d, ximg, wimg, want = _prefill_setup(nv, m, k, n, 11)
    pieces_d = cuda(pieces)
    lib = nv.lib()
    dt = torch.int8 if q8 else torch.bfloat16
    ck = torch.full((L, S1, H, T, D), 7, dtype=dt, device="cuda")
    cv = torch.full((L, S1, H, T, D), 7, dtype=dt, device="cuda")
    cks = torch.full((L, S1, H, T), -1.0, device="cuda") if q8 else None
    cvs = torch.full((L, S1, H, T), -1.0, device="cuda") if q8 else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    nv.check(lib.b200dec_prefill_gemm(nv.ptr(ximg), m, k, nv.ptr(wimg), nv.ptr(b_d), n, 2 if q8 else 1, None,
                                      nv.ptr(pieces_d), len(pieces), nv.ptr(ck), nv.ptr(cv), nv.ptr(cks), nv.ptr(cvs),
                                      L, S1, H, D, T, nv.ptr(status), nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    kv = want.reshape(m, L, 2, H, D)
    touched = np.zeros((S1, T), bool)
    for first, frames, slot, _ in pieces:
        touched[slot, :frames] = True
        for which, cache, scales in ((0, ck, cks), (1, cv, cvs)):
            ref = kv[first:first + frames, :, which].transpose(1, 2, 0, 3)  # (L, H, frames, D)
            got = cache[:, slot, :, :frames].float().cpu().numpy()
            if not q8:
                np.testing.assert_allclose(got, ref, atol=1e-4, rtol=2.0 ** -8)  # one bf16 rounding of a ~fp32 sum
            else:
                sc = scales[:, slot, :, :frames].cpu().numpy()
                rb = bf16_round(ref.astype(np.float32))
                np.testing.assert_allclose(sc, np.abs(rb).max(-1) / 127, rtol=2.0 ** -6)  # one bf16 step of the largest
                assert np.abs(got * sc[..., None] - rb).max() <= 0.51 * sc.max() + 2.0 ** -7 * np.abs(rb).max()
    for cache in (ck, cv):  # cells of no piece are untouched
        assert (cache.float().cpu().numpy().transpose(0, 2, 1, 3, 4)[:, :, ~touched] == 7).all()
    if q8:
        assert (cks.cpu().numpy().transpose(0, 2, 1, 3)[:, :, ~touched] == -1).all()


def test_read_probe_launches_and_checks_its_arguments(nv):
    """The measurement aid b200dec_read_probe: a launch that only reads; it must accept a graph capture, leave its sink
    alone and refuse sizes that are not whole 16-byte pieces."""
    lib = nv.lib()
    src = torch.arange(1 << 22, dtype=torch.int32, device="cuda")  # 16 MB
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    for pdl in (0, 1):
        nv.check(lib.b200dec_read_probe(nv.ptr(src), 256, 65536, nv.ptr(sink), pdl, nv.stream_ptr()))
    torch.cuda.synchronize()
    assert int(sink.item()) == 0
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        nv.check(lib.b200dec_read_probe(nv.ptr(src), 1024, 16384, None, 0, nv.stream_ptr(side)))
    graph.replay()
    torch.cuda.synchronize()
    assert lib.b200dec_read_probe(nv.ptr(src), 256, 65530, None, 0, nv.stream_ptr()) != 0
    assert lib.b200dec_read_probe(None, 256, 65536, None, 0, nv.stream_ptr()) != 0
    assert b"read_probe" in lib.b200dec_last_error()
