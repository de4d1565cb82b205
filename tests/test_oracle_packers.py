"""The numpy packers of oracle/packers.py against the reference's own functions' outputs (tests/golden/packers.npz,
made by tests/golden/make_golden.py from kernels/stream_decoder.py and kernels/sparse.py): bit-exact."""

import os

import numpy as np
import pytest

from oracle import packers


@pytest.fixture(scope="module")
def g(golden_dir):
    return np.load(os.path.join(golden_dir, "packers.npz"))


@pytest.mark.parametrize("case", ["a", "b", "c"])
def test_prepare_w8_bit_exact(g, case):
    u8, s = packers.prepare_w8(g[f"{case}_w"])
    assert u8.dtype == np.uint8 and np.array_equal(u8, g[f"{case}_u8"])
    assert np.array_equal(s.view(np.uint32), g[f"{case}_s"].view(np.uint32))
    q, _ = packers.quantize_rows(g[f"{case}_w"])
    assert np.array_equal(packers.unpermute_w8(u8), q)


@pytest.mark.parametrize("case", ["a", "b", "c"])
def test_prune_quantize_compress_bit_exact(g, case):
    pruned = packers.prune_24_magnitude(g[f"{case}_w"])
    if case != "a":  # case a holds exact ties, where the reference's choice is torch.topk's
        assert np.array_equal(pruned, g[f"{case}_pruned"])
    else:
        ties = np.zeros(pruned.shape[0], bool)
        ties[[3, 5]] = True
        assert np.array_equal(pruned[~ties], g["a_pruned"][~ties])
        assert ((pruned.reshape(pruned.shape[0], -1, 4) != 0).sum(-1) <= 2).all()
    qp, sp = packers.quantize_rows(g[f"{case}_pruned"])
    assert np.array_equal(qp, g[f"{case}_qp"]) and np.array_equal(sp, g[f"{case}_sp"])
    kept, words = packers.compress_24(g[f"{case}_qp"])
    assert np.array_equal(kept, g[f"{case}_kept"]) and np.array_equal(words, g[f"{case}_words"])
    assert np.array_equal(packers.expand_24(kept, words), g[f"{case}_qp"])


def test_compress_patterns(g):
    kept, words = packers.compress_24(g["p_q"])
    assert np.array_equal(kept, g["p_kept"]) and np.array_equal(words, g["p_words"])
    assert np.array_equal(packers.expand_24(g["p_kept"], g["p_words"]), g["p_q"])


def test_compress_rejects_dense():
    q = np.ones((1, 32), np.int8)
    with pytest.raises(AssertionError):
        packers.compress_24(q)


def test_fp16_image_keeps_the_bf16_values():
    """The 16-bit mode's weights, fp16(bf16(w)): every bf16 value of magnitude 2^-14 .. 65280 (the largest below the fp16 limit) bit for bit, the smaller
    ones within 2^-25 (the fp16 subnormal grid), and a weight beyond the fp16 range refused."""
    import torch
    from cohere_inference_b200.packing import fp16_image
    from oracle.decoder import bf16_round
    rng = np.random.default_rng(9)
    w = np.concatenate([rng.standard_normal(4096) * 0.02, rng.standard_normal(512) * 1e-5, rng.standard_normal(512) * 50,
                        [0.0, -0.0, 2.0 ** -14, -(2.0 ** -14), 2.0 ** -15, 65280.0, -65280.0]]).astype(np.float32)
    got = fp16_image(torch.from_numpy(w)).float().numpy()
    want = bf16_round(w)
    big = np.abs(want) >= 2.0 ** -14
    assert np.array_equal(got[big], want[big]) and big.sum() > 4500
    assert np.abs(got[~big] - want[~big]).max() <= 2.0 ** -25 and (~big).sum() > 400
    with pytest.raises(AssertionError, match="fp16 range"):
        fp16_image(torch.tensor([[0.5, 7e4]]))

