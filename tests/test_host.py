"""CPU-only checks: the C-ABI library exports what include/b200dec.h declares, the slot scheduler's invariants over the
CPU oracle (same API as StreamDecoder), the request stream, and the data-parallel partition + stats gather on two gloo
ranks."""

import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from cohere_inference_b200 import synthetic_model, synthetic_requests
from cohere_inference_b200.scheduler import DecodeScheduler
from oracle.decoder import OracleConfig, StreamOracle, effective_weights, state_to_numpy

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from cohere_inference_b200 import build, native
    build.build()
    header = open(os.path.join(ROOT, "include", "b200dec.h")).read()
    declared = set(re.findall(r"\b(b200dec_[a-z0-9_]+)\s*\(", header))
    assert declared == set(native.PROTOTYPES), declared ^ set(native.PROTOTYPES)
    lib = ctypes.CDLL(native.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert native.lib().b200dec_version() == 1
    # pure host queries need no GPU
    assert native.lib().b200dec_tiled_bytes(native.W_INT8_24, 1024, 4096) == 1024 * 4096 // 2
    assert native.lib().b200dec_attention_scratch_floats(64, 16, 64) == 64 * 16 * 16 * 66


def test_weight_kinds_sizes_and_tile_choices():
    """The pure host side of the seven weight kinds: bytes of the tiled images, which (kind, operand, tile) combinations
    have a kernel, and that packing.tile_config only hands out tiles the library accepts for the rows it was asked
    for (or, failing that, for two passes of 64)."""
    from cohere_inference_b200 import native as nv, packing as pk
    lib = nv.lib()
    n, k = 4096, 1024
    per_weight = {nv.W_BF16: 2, nv.W_F16: 2, nv.W_F16_UMMA: 2, nv.W_INT8: 1, nv.W_INT8_UMMA: 1, nv.W_INT8_24: 0.5,
                  nv.W_INT8_24_UMMA: 0.5}
    for kind, b in per_weight.items():
        assert lib.b200dec_tiled_bytes(kind, n, k) == int(n * k * b), kind
        sparse = kind in (nv.W_INT8_24, nv.W_INT8_24_UMMA)
        assert lib.b200dec_tiled_meta_bytes(kind, n, k) == (n * k // 8 if sparse else 0), kind
    assert lib.b200dec_tiled_bytes(99, n, k) == -1
    # the tcgen05 kinds: fp16 rows only (plain, or a LayerNorm's ready operand), K = 1024 split 4 or 8, K = 4096 split 8
    for kind in (nv.W_INT8_UMMA, nv.W_F16_UMMA, nv.W_INT8_24_UMMA):
        assert lib.b200dec_linear_fits(kind, nv.A_F16, 0, 8, 4, 1024, 128) == 1
        assert lib.b200dec_linear_fits(kind, nv.A_F16_ROWS16, 1, 8, 8, 1024, 64) == 1
        assert lib.b200dec_linear_fits(kind, nv.A_F16, 0, 8, 8, 4096, 128) == 1
        assert lib.b200dec_linear_fits(kind, nv.A_F16, 1, 8, 4, 1024, 64) == 0         # fp32 rows to normalise
        assert lib.b200dec_linear_fits(kind, nv.A_F32_SPLIT, 0, 8, 4, 1024, 64) == 0   # split operand
        assert lib.b200dec_linear_fits(kind, nv.A_F16_ROWS16, 1, 8, 8, 4096, 64) == 0  # no LayerNorm over K = 4096
        assert lib.b200dec_linear_fits(kind, nv.A_F16, 0, 8, 2, 1024, 64) == 0
    # the mma.sync kinds: the fp16 kind takes the int8 kinds' operands, the bf16 kind has no linked LayerNorm
    assert lib.b200dec_linear_fits(nv.W_F16, nv.A_F16_ROWS16, 1, 8, 4, 1024, 128) == 1
    assert lib.b200dec_linear_fits(nv.W_INT8, nv.A_F16_ROWS16, 1, 8, 4, 1024, 128) == 1
    assert lib.b200dec_linear_fits(nv.W_BF16, nv.A_F16_ROWS16, 1, 8, 4, 1024, 64) == 0
    for kind in (nv.W_INT8, nv.W_BF16, nv.W_F16, nv.W_INT8_24):
        a_kind = nv.A_F32_SPLIT if kind == nv.W_BF16 else nv.A_F16
        for shape in ((3072, 1024), (1024, 1024), (4096, 1024), (1024, 4096), (16384, 1024)):
            for ln in (False, True):
                if ln and shape[1] != 1024:
                    continue
                for rows in (1, 16, 64, 128):
                    w, s = pk.tile_config(*shape, kind, a_kind, ln, rows)
                    assert shape[0] % (16 * w) == 0 and shape[1] % s == 0
                    linked = ln and a_kind == nv.A_F16 and kind != nv.W_BF16 and shape[1] // s <= 256
                    q_kind = nv.A_F16_ROWS16 if linked else a_kind
                    fits = lambda r: lib.b200dec_linear_fits(kind, q_kind, int(ln), w, s, shape[1], r)  # noqa: E731
                    assert fits(rows) or fits(min(rows, 64)), (kind, shape, ln, rows, w, s)


def test_structs_match_header_sizes():
    from cohere_inference_b200 import native
    assert ctypes.sizeof(native.Weight) == 72 and ctypes.sizeof(native.Norm) == 24  # 6 pointers + 5 ints, padded
    assert ctypes.sizeof(native.Layer) == 3 * 24 + 6 * 72 + 8 * 8
    lib = native.lib()  # and every structure against the library as compiled
    for which, struct in enumerate((native.Weight, native.Norm, native.Layer, native.Plan, native.LnLink)):
        assert lib.b200dec_sizeof(which) == ctypes.sizeof(struct), struct.__name__


def test_missing_library_fails_loudly(monkeypatch):
    from cohere_inference_b200 import native
    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setattr(native, "LIB_PATH", "/nonexistent/libb200dec.so")
    with pytest.raises(native.NativeError, match="no PyTorch or CPU fallback"):
        native.lib()


def test_request_stream_is_seeded_and_keeps_slots_full():
    a, b = synthetic_requests(2000, seed=0), synthetic_requests(2000, seed=0)
    assert all(x.frames == y.frames and x.target == y.target and x.arrival == y.arrival and
               np.array_equal(x.prompt, y.prompt) for x, y in zip(a, b))
    assert min(r.frames for r in a) >= 50 and max(r.frames for r in a) <= 375
    assert min(r.target for r in a) >= 16 and max(r.target for r in a) <= 448
    rate = len(a) / a[-1].arrival  # requests per step
    assert abs(rate - 0.95 * 128 / 241) / rate < 0.05


@pytest.fixture(scope="module")
def tiny():
    model = synthetic_model(2, heads=2, head_dim=8, act="gelu", layers=1, hidden=16, ffn=32, vocab=40, max_pos=64)
    w = effective_weights(state_to_numpy(model), 1)
    return model, w


def _alone(w, cfg, r, mem, max_new):
    so = StreamOracle(w, cfg, slots=1, max_new_tokens=max_new, max_prompt=16, frames=64)
    so.fill_cross(mem, [r.frames], [0])
    so.admit([0], [r.prompt], [r.frames], [min(r.target, max_new)])
    b = so.set_active([0])
    while not so.finished[0]:
        so.step(b)
    return so.out[0].copy()


def test_scheduler_invariants_over_cpu_oracle(tiny):
    """Continuous batching is invisible in the results: every request decodes to the tokens it gets alone; slots are
    reused, never shared; a flag is only trusted after admission; eos ends a request early."""
    model, w = tiny
    cfg = OracleConfig.of(model.config)
    reqs = synthetic_requests(30, seed=3, vocab=40, prompt_len=4, frames=(2, 9), targets=(1, 12), slots=4, fill=1.5)
    mem = {r.mem_seed: np.random.default_rng(r.mem_seed).standard_normal((r.frames, 16)).astype(np.float32) for r in reqs}
    dec = StreamOracle(w, cfg, slots=4, max_new_tokens=12, max_prompt=16, frames=64)
    trace = []
    sched = DecodeScheduler(dec, lambda r: mem[r.mem_seed], trace=trace)
    got = sched.run(reqs)
    st = sched.stats
    assert st.admitted == st.evicted == 30 and sorted(sched.free) == [0, 1, 2, 3]
    ended_by_eos = 0
    for r, g in zip(reqs, got):
        row = _alone(w, cfg, r, mem[r.mem_seed], 12)
        gen = row[4:]
        end = np.nonzero(gen == dec.eos)[0]
        n = 4 + (end[0] + 1 if len(end) else min(r.target, 12))
        ended_by_eos += bool(len(end)) and end[0] + 1 < r.target
        assert np.array_equal(g, row[:n])
    live = set()
    for step, what, slots in trace:  # a slot is admitted only when free, evicted only when live
        for s in slots:
            assert (s not in live) if what == "admit" else (s in live)
            (live.add if what == "admit" else live.discard)(s)
    assert not live
    assert st.row_steps <= st.padded_row_steps <= st.slot_steps and st.steps > 0
    assert st.occupancy > 0.5
    assert st.delivered_tokens == sum(len(g) for g in got)


def test_scheduler_waits_for_a_free_slot(tiny):
    """Three requests, two slots: the third is admitted only after an eviction freed a slot. (Over the CPU oracle the
    flags are current as soon as a step returns, so no finished row is re-run; on a GPU the LAG-1 read re-runs it
    once, which the GPU tests cover.)"""
    model, w = tiny
    cfg = OracleConfig.of(model.config)
    reqs = synthetic_requests(3, seed=1, vocab=40, prompt_len=2, frames=(3, 3), targets=(2, 2), slots=2, fill=4.0)
    for r in reqs:
        r.arrival = 0.0
    mem = np.random.default_rng(0).standard_normal((3, 16)).astype(np.float32)
    dec = StreamOracle(w, cfg, slots=2, max_new_tokens=4, max_prompt=16, frames=64, eos=-1)
    sched = DecodeScheduler(dec, lambda r: mem)
    got = sched.run(reqs)
    assert all(len(g) == 4 for g in got)
    # 2 slots, 3 requests of 3 steps each: two run together, the third alone afterwards
    assert sched.stats.steps == 6 and sched.stats.row_steps == 9 and sched.stats.bucket_steps == {2: 3, 1: 3}


def test_data_parallel_partition_and_stats_gather_two_gloo_ranks(tmp_path):
    script = tmp_path / "dp.py"
    script.write_text(f"""
import sys
sys.path.insert(0, {ROOT!r})
import numpy as np
from cohere_inference_b200 import dataparallel as dp, synthetic_model, synthetic_requests
from cohere_inference_b200.scheduler import DecodeScheduler
from oracle.decoder import OracleConfig, StreamOracle, effective_weights, state_to_numpy
rank, local, world = dp.init("gloo")
assert world == 2
model = synthetic_model(2, heads=2, head_dim=8, layers=1, hidden=16, ffn=32, vocab=40, max_pos=64)
w = effective_weights(state_to_numpy(model), 1)
reqs = synthetic_requests(21, seed=4, vocab=40, prompt_len=3, frames=(2, 6), targets=(1, 8), slots=4)
mine = dp.partition(reqs, rank, world)
assert [r.mem_seed for r in mine] == [r.mem_seed for r in reqs[rank::2]]
dec = StreamOracle(w, OracleConfig.of(model.config), slots=4, max_new_tokens=8, max_prompt=16, frames=64, eos=-1)
sched = DecodeScheduler(dec, lambda r: np.random.default_rng(r.mem_seed).standard_normal((r.frames, 16)).astype(np.float32))
dp.barrier()
out = sched.run(mine)
st = sched.stats
all_stats = dp.gather_stats(dict(steps=st.steps, new_tokens=st.new_tokens, admitted=st.admitted, evicted=st.evicted))
assert len(all_stats) == 2 and all_stats[rank]["new_tokens"] == sum(r.target for r in mine)
assert sum(s["new_tokens"] for s in all_stats) == sum(r.target for r in reqs)
assert sum(s["admitted"] for s in all_stats) == 21
assert dp.max_over_ranks(float(rank)) == 1.0
sys.stdout.write("rank%d-ok\\n" % rank)
""")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29617", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "rank0-ok" in r.stdout and "rank1-ok" in r.stdout


def test_data_parallel_rank_failure_is_an_error_not_a_hang(tmp_path):
    """A rank that raises before the stats gather ends the job with an error on the host (no GPU involved)."""
    script = tmp_path / "dp_fail.py"
    script.write_text(f"""
import sys, datetime
sys.path.insert(0, {ROOT!r})
import torch.distributed as dist
from cohere_inference_b200 import dataparallel as dp
import os
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
if dist.get_rank() == 1:
    raise RuntimeError("injected failure before the gather")
dp.gather_stats(dict(steps=1))
""")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29618", str(script)],
                       capture_output=True, text=True, env=dict(os.environ, MASTER_ADDR="127.0.0.1"), timeout=120)
    assert r.returncode != 0 and "injected failure" in (r.stdout + r.stderr)
