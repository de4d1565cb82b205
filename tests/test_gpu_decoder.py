"""Whole-step parity on a B200: StreamDecoder (C-ABI kernels under CUDA graphs) against the fp32 oracle on the same
seeded weights and inputs. Tolerances are the ones the benchmark definition states: per-step logits within 2e-2
max-abs of the fp32 path on the weights the mode stores (dequantised int8 / bf16-rounded), greedy agreement >= 99.5 %
under teacher forcing."""

import os

import numpy as np
import pytest
import torch

from cohere_inference_b200.synth import config1_inputs, synthetic_model, synthetic_requests
from oracle.decoder import OracleConfig, StreamOracle, argmax_first, effective_weights, state_to_numpy

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2


@pytest.fixture(scope="module")
def model16():
    return synthetic_model(0)  # 16 heads x 64, GELU: the benchmark architecture


@pytest.fixture(scope="module")
def state16(model16):
    return state_to_numpy(model16)


def _decoder(model, **kw):
    from cohere_inference_b200 import StreamDecoder
    return StreamDecoder(model.cuda(), **kw)


def _run_teacher_forced(dec, memory, prompts, steps, slots=None):
    """Admit one request per row, step `steps` times; returns logits (steps, B, V) and argmax (steps, B)."""
    B = len(prompts)
    slots = slots or list(range(B))
    lengths = [m.shape[0] for m in memory]
    with torch.cuda.stream(dec.stream):
        dec.fill_cross(torch.from_numpy(np.concatenate(memory)).cuda(), lengths, slots)
    dec.admit(slots, [torch.from_numpy(p) for p in prompts], lengths)
    b = dec.set_active(slots)
    lg, am = [], []
    for _ in range(steps):
        dec.step(b)
        dec.stream.synchronize()
        lg.append(dec.logits[:B].cpu().numpy().copy())
        am.append(dec.argmax[slots].cpu().numpy().copy())
    dec.check_status()
    return np.stack(lg), np.stack(am)


def test_config1_bf16_against_transformers_golden(model16, golden_dir):
    """BASELINE config 1 on the GPU in bf16-weight mode against the transformers fp32 run (tests/golden): the golden
    logits are those of unrounded fp32 weights, so this also bounds what storing weights as bf16 costs."""
    g = np.load(os.path.join(golden_dir, "decoder_config1.npz"))
    memory, prompt = config1_inputs(0)
    dec = _decoder(model16, slots=4, max_new_tokens=64, max_prompt=16, max_audio_s=10.0, eos=-1, record=True)
    # teacher forcing with the golden's own tokens: prompt, then its greedy continuation
    seq = np.concatenate([prompt[0], g["argmax"][9:]])
    lg, am = [], []
    with torch.cuda.stream(dec.stream):
        dec.fill_cross(torch.from_numpy(memory[0]).cuda(), [125], [2])
    dec.admit([2], [torch.from_numpy(prompt[0])], [125])
    b = dec.set_active([2])
    for t in range(73):
        dec.step(b)
        dec.stream.synchronize()
        lg.append(dec.logits[0].cpu().numpy().copy())
        am.append(int(dec.argmax[2]))
        if t + 1 >= 10:  # past the prompt the decoder feeds its own choice: overwrite it with the golden token
            dec.tok[2] = int(seq[t + 1]) if t + 1 < len(seq) else 0
    lg = np.stack(lg)
    err = np.abs(lg[:, ::64] - g["logits_sub"]).max()
    agree = (np.array(am) == g["argmax"]).mean()
    print(f"config1 bf16: max-abs logit error {err:.2e}, greedy agreement {agree:.4f}")
    assert err <= LOGIT_TOL
    assert agree >= 0.97  # vs unrounded weights; the 99.5 % gate is on the stored weights (next tests)
    dec.check_status()


@pytest.mark.parametrize("mode,kw", [("bf16", {}), ("int8", dict(int8=True, umma_above_rows=0)),
                                     ("int8_small_buckets_on_mma_sync", dict(int8=True)),
                                     ("int8_24", dict(int8=True, ffn_sparse=True, umma_above_rows=0)),
                                     ("fp16", dict(fp16_weights=True)),
                                     ("fp16_umma_all", dict(fp16_weights=True, proj_umma="all", umma_above_rows=0)),
                                     ("fp16_no_umma", dict(fp16_weights=True, proj_umma=False, head_umma=False)),
                                     ("int8_kv8", dict(int8=True, kv_int8=True, umma_above_rows=0)),
                                     ("int8_umma_all", dict(int8=True, proj_umma="all", umma_above_rows=0)),
                                     ("int8_no_umma", dict(int8=True, proj_umma=False)),
                                     ("int8_24_no_umma", dict(int8=True, ffn_sparse=True, proj_umma=False))])
def test_ragged_batch_logits_and_greedy_agreement(model16, state16, mode, kw):
    """Five rows with different prompts, prompt lengths and encoder lengths (50..375), 40 steps, the padding rows of
    bucket 8 on the dummy slot; the oracle runs the weights the mode stores (and, for int8 caches, quantises its keys
    and values the same way)."""
    rng = np.random.default_rng(17)
    B, steps = 5, 40
    frames = [50, 375, 211, 125, 300]
    memory = [rng.standard_normal((t, 1024)).astype(np.float32) for t in frames]
    prompts = [rng.integers(0, 16384, n).astype(np.int64) for n in (10, 3, 16, 1, 10)]
    dec = _decoder(model16, slots=8, max_new_tokens=64, max_prompt=16, max_audio_s=30.0, eos=-1, record=True, **kw)
    slots = [5, 0, 7, 2, 3]
    lg, am = _run_teacher_forced(dec, memory, prompts, steps, slots)
    # the fp16 mode stores fp16(bf16(w)): the bf16 value itself wherever |w| >= 2^-14, within 2^-25 of it below
    w = effective_weights(state16, 8, "int8_24" if "24" in mode else "int8" if mode.startswith("int8") else "bf16", tables="bf16")
    so = StreamOracle(w, OracleConfig.of(model16.config), slots=8, max_new_tokens=64, max_prompt=16, frames=dec.frames,
                      kv_round="int8" if mode == "int8_kv8" else None, eos=-1, record=True)
    so.fill_cross(np.concatenate(memory), frames, slots)
    so.admit(slots, prompts, frames)
    ob = so.set_active(slots)
    # teacher forcing: the oracle is fed the GPU's tokens, so one flipped argmax does not derail the comparison
    out_gpu = dec.out.cpu().numpy()
    errs, agree = [], []
    for t in range(steps):
        so.step(ob)
        rec = so.record[-B:]
        want = np.stack([r[3] for r in rec])
        order = [slots.index(r[1]) for r in rec]
        errs.append(np.abs(lg[t][order] - want).max())
        agree.append(am[t][order] == argmax_first(want))
        for s in slots:  # force the GPU's token for the next step
            so.tok[s] = out_gpu[s, so.pos[s]]
            so.out[s, so.pos[s]] = out_gpu[s, so.pos[s]]
    err, rate = max(errs), np.mean(agree)
    print(f"{mode}: max-abs logit error {err:.2e}, greedy agreement {rate:.4f} over {B * steps} row-steps")
    assert err <= LOGIT_TOL
    assert rate >= 0.995
    assert np.array_equal(dec.pos.cpu().numpy()[slots], so.pos[slots])


def test_heads_8x128_relu(state16):
    """The reference's own head split and activation (8 heads x 128, ReLU) with nonzero biases and LayerNorm affines."""
    model = synthetic_model(3, heads=8, head_dim=128, act="relu", bias_std=0.05)
    rng = np.random.default_rng(4)
    frames = [60, 200]
    memory = [rng.standard_normal((t, 1024)).astype(np.float32) for t in frames]
    prompts = [rng.integers(0, 16384, 4).astype(np.int64) for _ in range(2)]
    dec = _decoder(model, slots=2, max_new_tokens=32, max_prompt=8, max_audio_s=20.0, eos=-1, record=True, int8=True)
    lg, am = _run_teacher_forced(dec, memory, prompts, 12)
    w = effective_weights(state_to_numpy(model), 8, "int8", tables="bf16")
    so = StreamOracle(w, OracleConfig.of(model.config), slots=2, max_new_tokens=32, max_prompt=8, frames=dec.frames,
                      eos=-1, record=True)
    so.fill_cross(np.concatenate(memory), frames, [0, 1])
    so.admit([0, 1], prompts, frames)
    ob = so.set_active([0, 1])
    out_gpu = dec.out.cpu().numpy()
    for t in range(12):
        so.step(ob)
        want = np.stack([r[3] for r in so.record[-2:]])
        assert np.abs(lg[t] - want).max() <= LOGIT_TOL
        for s in (0, 1):
            so.tok[s] = out_gpu[s, so.pos[s]]


def test_graph_replay_equals_direct_launch_and_is_deterministic(model16):
    rng = np.random.default_rng(2)
    memory = [rng.standard_normal((80, 1024)).astype(np.float32) for _ in range(3)]
    prompts = [rng.integers(0, 16384, 5).astype(np.int64) for _ in range(3)]
    outs = []
    for graphs, pdl in ((True, True), (False, True), (False, False), (True, True)):
        dec = _decoder(model16, slots=4, max_new_tokens=16, max_prompt=8, max_audio_s=10.0, eos=-1, record=True,
                       int8=True, graphs=graphs, pdl=pdl)
        lg, _ = _run_teacher_forced(dec, memory, prompts, 20)
        outs.append((lg, dec.out.cpu().numpy().copy()))
    for lg, out in outs[1:]:
        assert np.array_equal(lg, outs[0][0]) and np.array_equal(out, outs[0][1])


def test_eos_limit_and_finished_rows(model16):
    """A row ends at its token limit, keeps re-running its last position until evicted, and changes nothing."""
    rng = np.random.default_rng(8)
    memory = [rng.standard_normal((50, 1024)).astype(np.float32) for _ in range(2)]
    prompts = [rng.integers(0, 16384, 3).astype(np.int64) for _ in range(2)]
    dec = _decoder(model16, slots=2, max_new_tokens=16, max_prompt=8, max_audio_s=10.0, eos=-1, int8=True)
    with torch.cuda.stream(dec.stream):
        dec.fill_cross(torch.from_numpy(np.concatenate(memory)).cuda(), [50, 50], [0, 1])
    dec.admit([0, 1], [torch.from_numpy(p) for p in prompts], [50, 50], [4, 9])
    b = dec.set_active([0, 1])
    for _ in range(6):
        dec.step(b)
    dec.stream.synchronize()
    assert dec.flags.numpy()[:2].tolist() == [1, 0] and dec.pos.cpu().tolist()[:2] == [6, 6]
    snap = dec.out[0].cpu().numpy().copy()
    for _ in range(5):
        dec.step(b)
    dec.stream.synchronize()
    assert dec.flags.numpy()[:2].tolist() == [1, 1] and dec.pos.cpu().tolist()[:2] == [6, 11]
    assert np.array_equal(dec.out[0].cpu().numpy(), snap)
    assert (snap[:3] == prompts[0]).all() and (snap[7:] == dec.pad).all() and (snap[3:7] != dec.pad).all()
    dec.check_status()


def test_scheduler_stream_matches_oracle(model16, state16):
    """Continuous batching end to end: 12 requests through 4 slots (admission and eviction between replays, LAG-1 flag
    reads) give the same tokens as the CPU oracle decoding each request alone, up to near-tie flips."""
    from cohere_inference_b200 import DecodeScheduler
    reqs = synthetic_requests(12, seed=5, frames=(50, 120), targets=(4, 20), slots=4)
    mem = {r.mem_seed: np.random.default_rng(r.mem_seed).standard_normal((r.frames, 1024)).astype(np.float32)
           for r in reqs}
    dec = _decoder(model16, slots=4, max_new_tokens=32, max_prompt=16, max_audio_s=12.0, eos=-1, int8=True)
    trace = []
    sched = DecodeScheduler(dec, lambda r: torch.from_numpy(mem[r.mem_seed]), account_bytes=True, trace=trace)
    got = sched.run(reqs)
    dec.check_status()
    assert sched.stats.admitted == sched.stats.evicted == 12 and sorted(sched.free) == [0, 1, 2, 3]
    assert sched.stats.new_tokens == sum(r.target for r in reqs)
    w = effective_weights(state16, 8, "int8", tables="bf16")
    same = total = 0
    for i, r in enumerate(reqs):
        so = StreamOracle(w, OracleConfig.of(model16.config), slots=1, max_new_tokens=32, max_prompt=16, frames=dec.frames,
                          eos=-1)
        so.fill_cross(mem[r.mem_seed], [r.frames], [0])
        so.admit([0], [r.prompt], [r.frames], [r.target])
        b = so.set_active([0])
        while not so.finished[0]:
            so.step(b)
        want = so.out[0, :len(r.prompt) + r.target]
        assert len(got[i]) == len(want) and np.array_equal(got[i][:10], r.prompt)
        # compare up to the first divergence (a flipped near-tie changes everything after it)
        diff = np.nonzero(got[i] != want)[0]
        n = diff[0] if len(diff) else len(want)
        same += n - 10
        total += (n - 10) + (1 if len(diff) else 0)
    print(f"scheduler: {same}/{total} free-running tokens equal to the oracle before first divergence")
    assert same / total >= 0.98


@pytest.mark.parametrize("name,rows,kw", [("config3", 64, dict(int8=True)), ("config2", 8, dict()),
                                          ("config3_kv8", 64, dict(int8=True, kv_int8=True))])
def test_full_size_run_properties(model16, name, rows, kw):
    """The benchmark configurations at full size (10-token prompts + 448 new tokens = 457 steps; config 3: 64 rows,
    encoder lengths U[50, 375]; config 2: 8 rows of 375 frames), where the oracle is too slow. Size-independent
    properties instead: every row takes exactly plen - 1 + max_new steps and ends; the prompt is echoed; two runs give
    the same bits; and a row does not depend on its batch-mates: decoded alone and teacher-forced along the sequence
    it produced inside the batch (another bucket, so other tiles and summation orders), it picks the same next token
    at >= 99.5 % of the steps."""
    rng = np.random.default_rng(1000)
    new, plen = 448, 10
    frames = [375] * rows if name == "config2" else rng.integers(50, 376, rows).tolist()
    memory = [rng.standard_normal((t, 1024)).astype(np.float32) for t in frames]
    prompts = [rng.integers(0, 16384, plen).astype(np.int64) for _ in range(rows)]
    steps = plen - 1 + new
    outs = []
    for _ in range(2):
        dec = _decoder(model16, slots=rows, max_new_tokens=new, max_prompt=16, max_audio_s=30.0, eos=-1, **kw)
        slots = list(range(rows))
        with torch.cuda.stream(dec.stream):
            dec.fill_cross(torch.from_numpy(np.concatenate(memory)).cuda(), frames, slots)
        dec.admit(slots, [torch.from_numpy(p) for p in prompts], frames)
        b = dec.set_active(slots)
        for t in range(steps):
            dec.step(b)
            if t == steps - 2:
                dec.stream.synchronize()
                assert not dec.flags.numpy()[:rows].any()  # nobody ends early
        dec.stream.synchronize()
        dec.check_status()
        assert dec.flags.numpy()[:rows].all() and dec.pos.cpu().tolist()[:rows] == [steps] * rows
        out = dec.out[:rows].cpu().numpy().copy()
        assert all((out[r, :plen] == prompts[r]).all() for r in range(rows))
        assert (out[:, plen + new:] == dec.pad).all()
        outs.append(out)
        del dec
    assert np.array_equal(outs[0], outs[1])
    agree = []
    for r in (int(np.argmax(frames)), int(np.argmin(frames))):
        seq = outs[0][r, :plen + new]
        solo = _decoder(model16, slots=1, max_new_tokens=1, max_prompt=plen + new, max_audio_s=30.0, eos=-1,
                        record=True, **kw)
        _, am = _run_teacher_forced(solo, [memory[r]], [seq], steps, [0])
        agree.append((am[plen - 1:, 0] == seq[plen:]).mean())  # step t's un-forced choice is token t + 1
        del solo
    print(f"{name}: alone vs in the batch, greedy agreement {min(agree):.4f} over {new} steps")
    # int8 caches: a last-bit difference in a key can move its quantised value by a whole step, so near-ties flip more
    assert min(agree) >= (0.99 if kw.get("kv_int8") else 0.995)


@pytest.mark.parametrize("mode,kw,min_agree,max_err", [("int8", dict(int8=True), 0.85, 0.15),
                                                        ("int8_24", dict(int8=True, ffn_sparse=True), 0.0, 10.0)])
def test_config1_quantised_against_fp32_golden(model16, golden_dir, mode, kw, min_agree, max_err):
    """What the quantisation itself costs: BASELINE config 1 with int8 (and 2:4) weights against the transformers run
    on the ORIGINAL fp32 weights. The 2e-2 / 99.5 % bars of the other tests are against the weights a mode stores
    (the reference's own definition, dec_w8.cu:4-5); this one is reported, with a loose gate for dense int8 and none
    for 2:4 (magnitude pruning of random-init weights removes half of every feed-forward product)."""
    g = np.load(os.path.join(golden_dir, "decoder_config1.npz"))
    memory, prompt = config1_inputs(0)
    seq = np.concatenate([prompt[0], g["argmax"][9:]]).astype(np.int64)  # 10 + 64 golden tokens
    dec = _decoder(model16, slots=2, max_new_tokens=1, max_prompt=len(seq), max_audio_s=10.0, eos=-1, record=True, **kw)
    lg, am = _run_teacher_forced(dec, [memory[0]], [seq], 73, [1])
    err = np.abs(lg[:, 0, ::64] - g["logits_sub"]).max()
    agree = (am[:, 0] == g["argmax"]).mean()
    flips = g["top2_gap"][am[:, 0] != g["argmax"]]
    print(f"config1 {mode} vs fp32 weights: max-abs logit error {err:.2e}, greedy agreement {agree:.4f}; golden top-2 "
          f"gap: median {np.median(g['top2_gap']):.3f}, at the flipped steps {np.sort(flips)[:5]}")
    assert err <= max_err and agree >= min_agree


def test_admit_and_device_active_list_match_the_oracle(model16):
    """b200dec_admit through the public method (one packed copy, one kernel) leaves the slot state the reference's
    admit defines, and with device_sched the device's own active list follows admissions and ends."""
    from oracle.decoder import StreamOracle, OracleConfig
    dec = _decoder(model16, slots=6, max_new_tokens=8, max_prompt=5, max_audio_s=10.0, eos=-1, int8=True,
                   device_sched=True)
    so = StreamOracle({}, OracleConfig.of(model16.config), slots=6, max_new_tokens=8, max_prompt=5, frames=dec.frames,
                      eos=-1)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 16384, n).astype(np.int64) for n in (5, 1, 3)]
    slots, frames, new = [4, 0, 3], [50, 77, 126], [2, 8, 5]
    with torch.cuda.stream(dec.stream):
        dec.fill_cross(torch.randn(sum(frames), 1024, device="cuda"), frames, slots)
    dec.admit(slots, prompts, frames, new)
    so.admit(slots, prompts, frames, new)
    dec.stream.synchronize()
    for name in ("tok", "pos", "plen", "limit", "cross_len", "finished", "forced", "out"):
        got, want = getattr(dec, name).cpu().numpy(), getattr(so, name)
        keep = slots if name in ("tok", "plen", "limit", "forced", "out") else slice(None)
        assert np.array_equal(got[keep], want[keep]), name
    assert dec.flags.numpy()[slots].tolist() == [0, 0, 0]
    assert int(dec.n_active.item()) == 3 and dec.active.cpu().tolist()[:3] == slots
    # slot 4 ends after plen - 1 + 2 = 6 steps; the step that ends it also drops it from the device's list
    b = dec.bucket(3)
    for t in range(6):
        dec.step(b)
    dec.stream.synchronize()
    assert dec.flags.numpy()[4] == 1 and int(dec.live.item()) == 2
    assert dec.active.cpu().tolist()[:b] == [0, 3] + [dec.dummy] * (b - 2)
    dec.admit([5], [prompts[1]], [60], [3])  # appended behind the live rows
    dec.stream.synchronize()
    assert dec.active.cpu().tolist()[:3] == [0, 3, 5] and int(dec.n_active.item()) == 3
    dec.check_status()
    with pytest.raises(ValueError):
        dec.admit([9], [prompts[0]], [60])  # no such slot


@pytest.mark.parametrize("bit,what,slots,buckets,mode", [
    (1, "vocabulary projection", 4, None, dict(int8=True)),
    (1, "vocabulary projection, 128-row bucket (the streamed-operand kernel)", 128, (128,), dict(int8=True)),
    (2, "layer projections", 4, None, dict(int8=True, umma_above_rows=0)),
    (1, "vocabulary projection, fp16 weight tiles by bulk copy", 4, None, dict(fp16_weights=True)),
    (1, "vocabulary projection, fp16 weight tiles, 128-row bucket", 128, (128,), dict(fp16_weights=True)),
    (2, "layer projections, fp16 weight tiles by bulk copy", 4, None,
     dict(fp16_weights=True, proj_umma="qkv,fc1", umma_above_rows=0)),
    (2, "layer projections, 2:4 weights expanded to dense tiles", 4, None,
     dict(int8=True, ffn_sparse=True, proj_umma="fc1", umma_above_rows=0))])
def test_bounded_wait_runs_out_and_the_context_survives(bit, what, slots, buckets, mode):
    """The tcgen05 kernels bound every wait. With a short limit and the test-only `withhold` switch (the producer of
    a barrier is left out, nothing faults and nothing is in flight), the wait runs out: the kernel returns, the status
    word carries the time-out, check_status raises, and the next ordinary steps on the same context give the same
    bits as before."""
    from cohere_inference_b200 import native as nv
    model = synthetic_model(0, layers=2)
    rng = np.random.default_rng(5)
    memory = [rng.standard_normal((60, 1024)).astype(np.float32) for _ in range(3)]
    prompts = [rng.integers(0, 16384, 6).astype(np.int64) for _ in range(3)]
    dec = _decoder(model, slots=slots, buckets=buckets, max_new_tokens=8, max_prompt=8, max_audio_s=10.0, eos=-1,
                   record=True, graphs=False, **mode)
    want, _ = _run_teacher_forced(dec, memory, prompts, 4)
    dec.admit([0, 1, 2], [torch.from_numpy(p) for p in prompts], [60] * 3)
    dec.plan.wait_limit, dec.plan.withhold = 2048, bit
    dec.step(dec.set_active([0, 1, 2]))
    with pytest.raises(nv.NativeError, match="bounded wait"):
        dec.check_status()
    dec.plan.wait_limit, dec.plan.withhold = 0, 0
    with torch.cuda.stream(dec.stream):
        dec.status.zero_()
    got, _ = _run_teacher_forced(dec, memory, prompts, 4)
    assert np.array_equal(got, want), what


def test_small_buckets_point_at_the_mma_sync_packing():
    """Buckets of up to `umma_above_rows` rows run the second, mma.sync packing of the tcgen05 projections; larger ones
    the tcgen05 packing; with 0 there is one packing. Both sets multiply by the same int8 values and scales."""
    import ctypes as C
    from cohere_inference_b200 import native as nv
    model = synthetic_model(0, layers=2)
    run = dict(slots=32, max_new_tokens=8, max_prompt=8, max_audio_s=10.0, eos=-1, graphs=False)
    dec = _decoder(model, int8=True, ffn_sparse=True, **run)
    assert dec._small_rows == 16 and set(dec.layers[0].small) == {"qkv", "fc1"}
    ly = dec.layers[0]
    assert (ly.qkv.kind, ly.small["qkv"].kind) == (nv.W_INT8_UMMA, nv.W_INT8)
    assert (ly.fc1.kind, ly.small["fc1"].kind) == (nv.W_INT8_24_UMMA, nv.W_INT8_24)
    assert torch.equal(ly.qkv.scale, ly.small["qkv"].scale) and torch.equal(ly.fc1.scale, ly.small["fc1"].scale)
    where = lambda: C.addressof(dec.plan.layer.contents)  # noqa: E731
    for b in dec.buckets:
        dec._select_layers(b)
        assert where() == C.addressof(dec._layer_structs_small if b <= 16 else dec._layer_structs), b
    one = _decoder(model, int8=True, ffn_sparse=True, umma_above_rows=0, **run)
    assert one._small_rows == 0 and not one.layers[0].small and one._layer_structs_small is None
    assert {k for k in dec.packed_tensors() if ".small." in k} and not {k for k in one.packed_tensors() if ".small." in k}


@pytest.mark.parametrize("mode", [dict(int8=True, ffn_sparse=True), dict(fp16_weights=True)])
def test_packed_weights_round_trip(tmp_path, mode):
    """save_packed -> from_packed: the same digest, the same bits out of the step, without the original model; a
    changed byte is caught by the manifest's SHA-256."""
    from cohere_inference_b200 import StreamDecoder
    model = synthetic_model(0, layers=2)
    rng = np.random.default_rng(6)
    memory = [rng.standard_normal((70, 1024)).astype(np.float32) for _ in range(3)]
    prompts = [rng.integers(0, 16384, 4).astype(np.int64) for _ in range(3)]
    run = dict(slots=4, max_new_tokens=8, max_prompt=8, max_audio_s=10.0, eos=-1, record=True)
    dec = _decoder(model, **mode, **run)
    want, _ = _run_teacher_forced(dec, memory, prompts, 5)
    path = str(tmp_path / "decoder.b200dec")
    digest = dec.save_packed(path)
    assert digest == dec.weights_digest() and len(digest) == 64
    del dec
    again = StreamDecoder.from_packed(path, **run)
    assert again.weights_digest() == digest and again.model is None
    assert again.fp16_weights == bool(mode.get("fp16_weights")) and again.int8 == bool(mode.get("int8"))
    got, _ = _run_teacher_forced(again, memory, prompts, 5)
    assert np.array_equal(got, want)
    blob = torch.load(path, weights_only=True)
    blob["tensors"]["layer1.fc2.tiled"][123] ^= 1
    torch.save(blob, path)
    with pytest.raises(ValueError, match="SHA-256"):
        StreamDecoder.from_packed(path, **run)
    with pytest.raises(ValueError, match="packed with"):  # tiled for buckets up to 4 rows, asked for up to 2
        StreamDecoder.from_packed(path, **dict(run, slots=2))


@pytest.mark.parametrize("style,shards", [("original", 3), ("module", 1)])
def test_decoder_from_a_checkpoint_directory(tmp_path, style, shards):
    """StreamDecoder.from_checkpoint reads config.json + *.safetensors (the names a published checkpoint carries, or
    the module names; one file or shards) and builds the same decoder as the module does: same digest of the packed
    weights, same bits out of the step. The real model's shape: 8 heads of 128, ReLU, 1280-wide encoder frames."""
    from cohere_inference_b200 import StreamDecoder
    from test_checkpoint import original_names, write_checkpoint
    model = synthetic_model(4, heads=8, head_dim=128, act="relu", layers=2, bias_std=0.05, dtype=torch.bfloat16)
    torch.manual_seed(1)
    model.model.decoder.proj = torch.nn.Linear(1280, 1024).to(torch.bfloat16).requires_grad_(False)
    model.config.encoder_hidden_size = 1280
    write_checkpoint(str(tmp_path), model, names=original_names() if style == "original" else None, shards=shards,
                     encoder_hidden=1280)
    rng = np.random.default_rng(8)
    memory = [rng.standard_normal((n, 1280)).astype(np.float32) for n in (70, 33, 101)]
    prompts = [rng.integers(0, 16384, 4).astype(np.int64) for _ in range(3)]
    run = dict(slots=4, max_new_tokens=8, max_prompt=8, max_audio_s=10.0, eos=-1, record=True, int8=True)
    dec = _decoder(model, **run)
    want, _ = _run_teacher_forced(dec, memory, prompts, 5)
    digest = dec.weights_digest()
    del dec
    again = StreamDecoder.from_checkpoint(str(tmp_path), **run)
    assert again.weights_digest() == digest
    assert (again.h, again.d, again.proj.k) == (8, 128, 1280)
    got, _ = _run_teacher_forced(again, memory, prompts, 5)
    assert np.array_equal(got, want)
